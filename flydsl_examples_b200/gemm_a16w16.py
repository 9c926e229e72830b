"""Host side of the B200 A16W16 GEMM: the reference's public call, kept as a drop-in.

    gemm_a16w16(a, b, out=None, bias=None, user_kwargs={}, stream=None, layout="nt", out_dtype=None)

mirrors kernels/gemm_a16w16_gfx950.py:1288-1441 of xytpai/flydsl-examples: same argument meaning, same
exception types and message prefixes. Underneath it makes one ctypes call into libb200_gemm.so
(hand-written sm_100a CUDA); there is no Triton, no torch.matmul and no CPU path here.

Accepted inputs are a superset of the reference's: operands whose base or leading stride is not 16-byte
aligned, 't' A with M not divisible by 8, and any K (K tails) all run. Pass
``user_kwargs["strict_reference_envelope"]=True`` to get the reference's rejections instead.
"""
from __future__ import annotations

import dataclasses

import ctypes as C
import threading
from collections import OrderedDict
from typing import Optional

import torch

from . import _lib
from . import policy as _policy

GEMM_A16W16_DTYPE_FP32 = _lib.DTYPE_FP32
GEMM_A16W16_DTYPE_BF16 = _lib.DTYPE_BF16
GEMM_A16W16_DTYPE_FP16 = _lib.DTYPE_FP16

# The reference's 16-byte DMA granule (kernels/gemm_a16w16_gfx950_utils.py:14); TMA has the same granule.
DMA_BYTES = 16

_STATUS_WORDS = 4
_ws_lock = threading.Lock()
_workspaces: dict[tuple, "_Workspace"] = {}
_sm_count: dict[int, int] = {}


class _Workspace:
    """Scratch owned by one (device, stream): split-K tickets + fp32 partial tiles + repack images, and the
    4-word status block kernels write when a bounded wait gives up. Grows on demand, never shrinks.
    Takes the place of get_split_k_buffers (kernels/gemm_a16w16_gfx950.py:1277-1281)."""

    __slots__ = ("buf", "status", "generation")

    def __init__(self, device: torch.device):
        self.buf = None
        self.generation = 0
        self.status = torch.zeros(_STATUS_WORDS, dtype=torch.int32, device=device)

    def ensure(self, nbytes: int, device: torch.device, stream: torch.cuda.Stream) -> None:
        if self.buf is None or self.buf.numel() < nbytes:
            with torch.cuda.stream(stream):
                # Zero-filled: the ticket area must start at zero; kernels leave it zero.
                self.buf = torch.zeros(max(nbytes, 4 << 20), dtype=torch.uint8, device=device)
            self.generation += 1  # prepared launches that point into the old buffer are stale


def _workspace_for(device: torch.device, stream: torch.cuda.Stream) -> _Workspace:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    with _ws_lock:
        ws = _workspaces.get(key)
        if ws is None:
            ws = _Workspace(device)
            _workspaces[key] = ws
        return ws


def _num_sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _sm_count[idx] = n
    return n


def _dtype_id(dt: torch.dtype) -> int:
    if dt is torch.float32:
        return GEMM_A16W16_DTYPE_FP32
    if dt is torch.bfloat16:
        return GEMM_A16W16_DTYPE_BF16
    if dt is torch.float16:
        return GEMM_A16W16_DTYPE_FP16
    raise AssertionError(f"unsupported dtype {dt}")


def _dtype_name(dt: torch.dtype) -> str:
    return {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}[dt]


def _check_operand(name: str, t: torch.Tensor, transposed: bool, strict: bool, m_for_a: Optional[int]) -> None:
    """Stride contract of one operand. Mirrors kernels/gemm_a16w16_gfx950.py:1322-1372: the contiguous
    dimension must have stride 1; in strict mode also the reference's 16-byte rules."""
    es = t.element_size()
    if transposed:
        bad = t.stride(0) != 1
        lead = t.stride(1)
        kind = "column-major"
        want = "stride(0) == 1"
    else:
        bad = t.stride(1) != 1
        lead = t.stride(0)
        kind = "row-major"
        want = "stride(1) == 1"
    extra = ""
    if strict:
        bad = bad or t.data_ptr() % DMA_BYTES != 0 or (lead * es) % DMA_BYTES != 0
        if name == "A" and transposed and m_for_a is not None:
            vec = DMA_BYTES // es
            bad = bad or m_for_a % vec != 0
            extra = f", and M divisible by {vec}"
        want += f" and a {DMA_BYTES}-byte-aligned data pointer and leading stride"
    if bad:
        raise ValueError(
            f"{name} does not satisfy the layout requirements for a {kind} input: expected {want}{extra}; "
            f"got shape={tuple(t.shape)} and stride={t.stride()}"
        )


def _strict_k_checks(k: int, kwargs: dict) -> None:
    """The reference's K-partition rules (kernels/gemm_a16w16_gfx950.py:1239-1274), applied only in strict
    mode: every split must be a whole number of block_k tiles, at least stages-1 of them, and an even count of
    at least two for its half-tile-interleaved kernel. The B200 kernels have none of these limits."""
    block_k = int(kwargs["block_k"])
    split_k = int(kwargs["split_k"])
    stages = int(kwargs["stages"])
    hti = bool(kwargs["use_half_tile_interleaved"])
    granule = DMA_BYTES // 2
    per_split = -(-k // split_k)
    per_split = -(-per_split // granule) * granule
    last = k - (split_k - 1) * per_split
    assert per_split % block_k == 0, (
        f"K-tail is unsupported: split-K partition of {per_split} elements is not a multiple of block_k={block_k}"
    )
    assert last > 0 and last % block_k == 0, (
        f"K-tail is unsupported: last split-K partition of {last} elements must be a positive multiple of "
        f"block_k={block_k}"
    )
    need = stages - 1
    for span, which in ((per_split, "each"), (last, "the last")):
        tiles = span // block_k
        assert tiles >= need, f"{which} split-K partition needs at least {need} K tiles, got {tiles}"
        if hti:
            assert tiles >= 2 and tiles % 2 == 0, (
                f"HTI requires at least two K tiles, and an even count, in {which} split-K partition; got {tiles}"
            )


def resolve_policy(m: int, n: int, k: int, dtype: torch.dtype, layout: str, user_kwargs: dict,
                   num_sms: int = _policy.NUM_SMS_DEFAULT, out_dtype: Optional[torch.dtype] = None) -> _policy.Policy:
    """user_kwargs -> Policy. A dict that names no tiling (empty, or control keys only) first consults the tuned
    JSONL, then the heuristic. The table and the heuristic are measured with 16-bit outputs; for an fp32 output
    (`out_dtype`) their pair tiles wider than 256 columns become 256 wide, because that variant's epilogue, which no main
    loop hides, takes twice as long with fp32 rows."""
    def for_output(pol: _policy.Policy) -> _policy.Policy:
        if out_dtype is torch.float32 and pol.cta_group == 2 and pol.tile_n > 256:
            return dataclasses.replace(pol, tile_n=256, stages=0)
        return pol

    if not any(key in user_kwargs for key in _policy.REFERENCE_KEYS + _policy.BLACKWELL_KEYS):
        rec = _policy.tuned_lookup(_dtype_name(dtype), layout, m, n, k)
        if rec is not None:
            control = {key: val for key, val in user_kwargs.items() if key in _policy.CONTROL_KEYS}
            pol = for_output(_policy.from_user_kwargs({**rec, **control}, m, n, k, layout, num_sms))
            if _policy.validate(pol, m, n, k, layout) is None:  # a row tuned for another layout may not fit this one
                return pol
    pol = _policy.from_user_kwargs(user_kwargs, m, n, k, layout, num_sms)
    return pol if "tile_n" in user_kwargs else for_output(pol)


def make_gemm_a16w16_param_and_validate(m: int, n: int, k: int, kwargs: dict):
    """Shape-dependent policy check: returns the resolved Policy, or None when it cannot run.
    Same role and name as kernels/gemm_a16w16_gfx950.py:1213-1236 (used by the tuner to filter configs)."""
    layout = ("t" if kwargs.get("a_is_transposed", False) else "n") + ("t" if kwargs.get("b_is_transposed", True) else "n")
    user = {key: val for key, val in kwargs.items()
            if key in _policy.REFERENCE_KEYS or key in _policy.BLACKWELL_KEYS}
    try:
        pol = _policy.from_user_kwargs(user, m, n, k, layout)
    except (ValueError, TypeError):
        return None
    return pol if _policy.validate(pol, m, n, k, layout) is None else None


_trace_buffer: Optional[torch.Tensor] = None


def set_trace_buffer(buf: Optional[torch.Tensor]) -> None:
    """Profiling aid: while set (a CUDA int64 tensor of at least grid*256 elements), every newly prepared call
    records per-CTA role timelines into it (see `trace` in include/b200_gemm.h). Pass None to turn it off."""
    global _trace_buffer
    _trace_buffer = buf
    clear_prepared_calls()


def _fill_args(a, b, out, bias, pol: _policy.Policy, a_t: bool, b_t: bool) -> _lib.Args:
    m, k = a.shape
    n = b.shape[1]
    args = _lib.Args()
    args.a = a.data_ptr()
    args.b = b.data_ptr()
    args.out = out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.m, args.n, args.k = m, n, k
    args.lda = a.stride(1) if a_t else a.stride(0)
    args.ldb = b.stride(1) if b_t else b.stride(0)
    # A stride of a size-1 dimension is arbitrary in torch; any value >= the extent describes the same memory.
    min_lda = m if a_t else k
    min_ldb = k if b_t else n
    if args.lda < min_lda:
        args.lda = min_lda
    if args.ldb < min_ldb:
        args.ldb = min_ldb
    args.ldo = n
    args.a_trans = 1 if a_t else 0
    args.b_trans = 1 if b_t else 0
    args.in_dtype = _dtype_id(a.dtype)
    args.out_dtype = _dtype_id(out.dtype)
    p = args.policy
    p.tile_n = pol.tile_n
    p.stages = pol.stages
    p.split_k = pol.split_k
    p.group_m = pol.group_m
    p.swap_ab = 1 if pol.swap_ab else 0
    p.cta_group = pol.cta_group
    p.split_mode = _policy.SPLIT_MODES[pol.split_mode]
    p.max_ctas = pol.max_ctas
    p.stream_k = 1 if pol.stream_k else 0
    p.no_pdl = 0 if pol.pdl else 1
    p.tile_k = pol.tile_k
    p.wait_limit_us = pol.wait_limit_us
    p.loader = 1 if pol.loader else 0
    return args


class _Prepared:
    """A resolved call kept for reuse: the C handle plus what it depends on."""

    __slots__ = ("handle", "ws", "ws_gen", "dev", "n")

    def __init__(self, handle, ws, dev, n):
        self.handle, self.ws, self.ws_gen, self.dev, self.n = handle, ws, ws.generation, dev, n


_PREPARED_MAX = 2048
_prepared: "OrderedDict[tuple, _Prepared]" = OrderedDict()
_prepared_lock = threading.Lock()


def _call_key(a, b, out, bias, kw_key, stream_ptr, layout, out_dtype):
    return (
        a.data_ptr(), a.shape, a.stride(), a.dtype,
        b.data_ptr(), b.shape, b.stride(),
        out.data_ptr(), out.shape, out.stride(), out.dtype,
        None if bias is None else (bias.data_ptr(), bias.shape, bias.stride(), bias.dtype),
        kw_key, stream_ptr, layout, out_dtype, a.device.index, b.dtype, b.device.index, out.device.index,
    )


def _remember(key, ent: _Prepared) -> None:
    with _prepared_lock:
        old = _prepared.pop(key, None)
        _prepared[key] = ent
        evicted = [old] if old is not None else []
        while len(_prepared) > _PREPARED_MAX:
            evicted.append(_prepared.popitem(last=False)[1])
    lib = _lib.load()
    for e in evicted:
        lib.b200_gemm_release(e.handle)


def clear_prepared_calls() -> None:
    """Drop every cached launch handle (tests; or after freeing the tensors they point at in bulk)."""
    with _prepared_lock:
        items = list(_prepared.values())
        _prepared.clear()
    lib = _lib.load()
    for e in items:
        lib.b200_gemm_release(e.handle)


def gemm_a16w16(
    a: torch.Tensor,
    b: torch.Tensor,
    out: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    user_kwargs: dict = {},
    stream: Optional[torch.cuda.Stream] = None,
    layout: str = "nt",
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Compute C[M, N] = A[M, K] @ B[K, N] (+ bias[N]) with fp32 accumulation and one final cast.

    Logical shapes never change with `layout`; each character only states which dimension of that operand is
    contiguous ('n' row-major, 't' column-major), exactly as in the reference. `out` may be any contiguous
    tensor with M*N elements; the returned tensor shares its storage. Asynchronous on `stream`.

    A call whose tensors (address, shape, strides, dtype), policy and stream were seen before reuses its resolved
    launch: validation, planning and tensor-map encoding are done once per distinct call.
    """
    # ---- repeat of a call seen before: one dictionary lookup and one C call
    if out is not None and a.is_cuda:
        stream_ptr = (torch.cuda.current_stream(a.device) if stream is None else stream).cuda_stream
        kw_key = tuple(sorted(user_kwargs.items())) if user_kwargs else ()
        key = _call_key(a, b, out, bias, kw_key, stream_ptr, layout, out_dtype)
        # The lock is held from the lookup to the end of the launch: a handle is released only after it has left the
        # table under the same lock, so none can be freed while a launch is reading it.
        with _prepared_lock:
            ent = _prepared.get(key)
            hit = ent is not None and ent.ws_gen == ent.ws.generation
            if hit:
                if torch.cuda.current_device() == ent.dev:
                    rc = _lib.load().b200_gemm_launch(ent.handle, stream_ptr)
                else:
                    with torch.cuda.device(ent.dev):
                        rc = _lib.load().b200_gemm_launch(ent.handle, stream_ptr)
        if hit:
            if rc != 0:
                raise RuntimeError(f"b200_gemm_launch failed ({rc}): {_lib.strerror(rc)}")
            return out.view(-1, ent.n)
    else:
        key = None

    # ---- first time: validate (same contract as the reference), plan, prepare, launch
    layout = layout.lower()
    if layout not in ("nn", "nt", "tn", "tt"):
        raise ValueError(f"unsupported GEMM layout: {layout!r}; expected 'nn', 'nt', 'tn', or 'tt'")
    a_t = layout[0] == "t"
    b_t = layout[1] == "t"
    device = a.device
    assert a.device == b.device
    assert a.ndim == 2 and b.ndim == 2
    m, k = a.shape
    assert b.shape[0] == k
    n = b.shape[1]
    assert a.dtype == b.dtype
    assert a.dtype in (torch.float16, torch.bfloat16)

    strict = bool(user_kwargs.get("strict_reference_envelope", False))
    _check_operand("A", a, a_t, strict, m)
    _check_operand("B", b, b_t, strict, None)

    if out_dtype is None:
        out_dtype = a.dtype if out is None else out.dtype
    if out_dtype not in (a.dtype, torch.float32):
        raise ValueError(f"unsupported output dtype {out_dtype}; expected {a.dtype} or torch.float32")
    out_in = out
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=device)
    else:
        assert out.dtype == out_dtype
        assert out.device == device
        assert out.is_contiguous()
    out = out.view(-1, n)
    assert out.shape[0] == m

    bias_in = bias
    if bias is not None:
        if not bias.is_contiguous():
            bias = bias.contiguous()
        assert bias.shape[0] == n
        assert bias.dtype == a.dtype

    if strict:
        merged = {"block_k": 64, "stages": 2, "split_k": 1, "k_waves": 1, "use_half_tile_interleaved": True}
        merged.update(user_kwargs)
        _strict_k_checks(k, merged)

    assert a.is_cuda, "gemm_a16w16 runs on CUDA tensors only (there is no CPU path)"
    if stream is None:
        stream = torch.cuda.current_stream(device)
    if m == 0 or n == 0:
        return out
    if k == 0:
        with torch.cuda.stream(stream):
            if bias is None:
                out.zero_()
            else:
                out.copy_(bias.to(out.dtype).expand(m, n))
        return out

    pol = resolve_policy(m, n, k, a.dtype, layout, user_kwargs, _num_sms(device), out_dtype)
    why = _policy.validate(pol, m, n, k, layout)
    assert why is None, f"unsupported gemm_a16w16 shape/config: {why}"

    args = _fill_args(a, b, out, bias, pol, a_t, b_t)
    lib = _lib.load()
    ws = _workspace_for(device, stream)
    dev_index = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev_index):
        need = lib.b200_gemm_workspace_bytes(C.byref(args))
        if need:
            ws.ensure(need, device, stream)
            args.workspace = ws.buf.data_ptr()
            args.workspace_bytes = ws.buf.numel()
        args.status = ws.status.data_ptr()
        if _trace_buffer is not None:
            args.trace = _trace_buffer.data_ptr()
            args.trace_words = _trace_buffer.numel()
        handle = C.c_void_p()
        rc = lib.b200_gemm_prepare(C.byref(args), C.byref(handle))
        if rc != 0:
            raise RuntimeError(f"b200_gemm_prepare failed ({rc}): {_lib.strerror(rc)}")
        rc = lib.b200_gemm_launch(handle, C.c_void_p(stream.cuda_stream))
    if rc != 0:
        lib.b200_gemm_release(handle)
        raise RuntimeError(f"b200_gemm_launch failed ({rc}): {_lib.strerror(rc)}")
    # Remember the launch only when it describes the caller's own tensors (a made-contiguous bias is a temporary).
    if key is not None and bias is bias_in and out_in is not None:
        _remember(key, _Prepared(handle, ws, dev_index, n))
    else:
        lib.b200_gemm_release(handle)
    return out


def gemm_a16w16_to_pointer(a: torch.Tensor, b: torch.Tensor, out_ptr: int, out_dtype: torch.dtype, user_kwargs: dict = {},
                           stream: Optional[torch.cuda.Stream] = None, layout: str = "nt") -> None:
    """The same product as `gemm_a16w16` (no bias), written to the raw device address `out_ptr`: an M x N
    row-major contiguous image of `out_dtype` that kernels on a's device can store to. This is how the fused
    K-sharded mode lets the epilogue write its tiles straight into another GPU's receive buffer over NVLink
    (`out_ptr` then comes from b200_peer_open). The caller owns the memory behind `out_ptr` and its lifetime."""
    layout = layout.lower()
    assert layout in ("nn", "nt", "tn", "tt") and a.is_cuda and a.device == b.device and a.dtype == b.dtype
    assert out_dtype in (a.dtype, torch.float32) and out_ptr % 16 == 0
    device = a.device
    if stream is None:
        stream = torch.cuda.current_stream(device)
    kw_key = tuple(sorted(user_kwargs.items())) if user_kwargs else ()
    key = ("ptr", a.data_ptr(), a.shape, a.stride(), a.dtype, b.data_ptr(), b.shape, b.stride(), out_ptr, out_dtype,
           kw_key, stream.cuda_stream, layout, device.index)
    lib = _lib.load()
    dev_index = device.index if device.index is not None else torch.cuda.current_device()
    with _prepared_lock:  # held across lookup and launch, see gemm_a16w16
        ent = _prepared.get(key)
        if ent is not None and ent.ws_gen == ent.ws.generation:
            with torch.cuda.device(ent.dev):
                rc = lib.b200_gemm_launch(ent.handle, C.c_void_p(stream.cuda_stream))
            if rc != 0:
                raise RuntimeError(f"b200_gemm_launch failed ({rc}): {_lib.strerror(rc)}")
            return
    a_t, b_t = layout[0] == "t", layout[1] == "t"
    m, k = a.shape
    n = b.shape[1]
    assert b.shape[0] == k and m > 0 and n > 0 and k > 0
    _check_operand("A", a, a_t, False, m)
    _check_operand("B", b, b_t, False, None)
    pol = resolve_policy(m, n, k, a.dtype, layout, user_kwargs, _num_sms(device), out_dtype)
    why = _policy.validate(pol, m, n, k, layout)
    assert why is None, f"unsupported gemm_a16w16 shape/config: {why}"
    args = _fill_args(a, b, torch.empty(0, dtype=out_dtype), None, pol, a_t, b_t)
    args.out = out_ptr
    ws = _workspace_for(device, stream)
    with torch.cuda.device(dev_index):
        need = lib.b200_gemm_workspace_bytes(C.byref(args))
        if need:
            ws.ensure(need, device, stream)
            args.workspace = ws.buf.data_ptr()
            args.workspace_bytes = ws.buf.numel()
        args.status = ws.status.data_ptr()
        handle = C.c_void_p()
        rc = lib.b200_gemm_prepare(C.byref(args), C.byref(handle))
    if rc != 0:
        raise RuntimeError(f"b200_gemm_prepare failed ({rc}): {_lib.strerror(rc)}")
    ent = _Prepared(handle, ws, dev_index, n)
    with torch.cuda.device(ent.dev):
        rc = lib.b200_gemm_launch(ent.handle, C.c_void_p(stream.cuda_stream))
    _remember(key, ent)  # only now can another thread find (and, by eviction, release) the handle
    if rc != 0:
        raise RuntimeError(f"b200_gemm_launch failed ({rc}): {_lib.strerror(rc)}")


def plan(a: torch.Tensor, b: torch.Tensor, layout: str = "nt", user_kwargs: dict = {},
         out_dtype: Optional[torch.dtype] = None, bias: Optional[torch.Tensor] = None) -> dict:
    """What a call with these arguments would launch (tile, stages, grid, workspace, repack flags)."""
    layout = layout.lower()
    a_t, b_t = layout[0] == "t", layout[1] == "t"
    m, k = a.shape
    n = b.shape[1]
    out_dtype = out_dtype or a.dtype
    pol = resolve_policy(m, n, k, a.dtype, layout, user_kwargs, out_dtype=out_dtype)
    fake_out = torch.empty(0, dtype=out_dtype)
    args = _fill_args(a, b, fake_out, bias, pol, a_t, b_t)
    pl = _lib.Plan()
    rc = _lib.load().b200_gemm_plan_query(C.byref(args), C.byref(pl))
    if rc != 0:
        raise RuntimeError(f"b200_gemm_plan_query failed ({rc}): {_lib.strerror(rc)}")
    return pl.as_dict()


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel launched through gemm_a16w16 on `device` abandoned a bounded wait."""
    torch.cuda.synchronize(device)
    with _ws_lock:
        items = list(_workspaces.items())
    for (dev, _stream), ws in items:
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        st = ws.status.tolist()
        if st[0] != 0:
            # A kernel that gave up may have left split-K / stream-K tickets taken: the next call on this workspace
            # would elect the wrong last arriver. Clear them, and forget every resolved launch.
            ws.status.zero_()
            if ws.buf is not None:
                ws.buf[: _lib.COUNTER_BYTES].zero_()
            torch.cuda.synchronize(ws.status.device)
            clear_prepared_calls()
            raise RuntimeError(f"b200 gemm kernel gave up a bounded wait: code={st[0]} cta={st[1]} role={st[2]} unit={st[3]}")

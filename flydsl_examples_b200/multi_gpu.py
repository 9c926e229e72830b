"""Single-box multi-GPU partitioning of one large GEMM (one process per GPU, torch.distributed for plumbing).

Three modes, none present in the reference (xytpai/flydsl-examples is single-GPU; its op is
kernels/gemm_a16w16_gfx950.py:1288):

  N-shard  rank r owns B[:, n0:n1] and computes C[:, n0:n1]. A is replicated. No communication at all.
  K-shard  rank r owns A[:, k0:k1] and B[k0:k1, :], computes a full-size fp32 partial product with the same CUDA
           kernel (fp32-output path), and the partials are summed across GPUs with an NCCL reduce-scatter over
           NVLink, chunk by chunk along M so the reduce of chunk i overlaps the GEMM of chunk i+1. Each rank ends up
           with 1/world of the rows of every chunk, rounded once (bias added) by a small cast kernel.

  fused K-shard  the same partition, but every rank's GEMM epilogue stores its fp32 tiles straight into the owning
           rank's receive slots over NVLink (peer memory) and the owner sums its slots; no collective moves data.

`gemm_fn` is the product call everywhere; the CPU tests inject their own function to exercise the partition and
exchange logic with gloo ranks.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import _lib

SHARD_ALIGN = 256  # shard boundaries fall on multiples of the widest tile where the size allows


def shard_bounds(extent: int, world: int, rank: int, align: int = SHARD_ALIGN) -> tuple[int, int]:
    """[begin, end) of `rank`'s slab of `extent`: as even as possible in units of `align`; the last ranks may
    get less (or nothing) when extent is small."""
    assert 0 <= rank < world
    units = -(-extent // align)
    base, rem = divmod(units, world)
    begin_u = rank * base + min(rank, rem)
    end_u = begin_u + base + (1 if rank < rem else 0)
    return min(begin_u * align, extent), min(end_u * align, extent)


def shard_b_along_n(b: torch.Tensor, world: int, rank: int) -> tuple[torch.Tensor, int, int]:
    """View of B[K, N] (any layout) restricted to this rank's columns. For an 'nt' B (stored [N, K]) that is a
    contiguous slab of rows of the stored matrix: a plain pointer offset, no copy."""
    n0, n1 = shard_bounds(b.shape[1], world, rank)
    return b[:, n0:n1], n0, n1


def shard_along_k(a: torch.Tensor, b: torch.Tensor, world: int, rank: int, align: int = 64):
    """Views A[:, k0:k1], B[k0:k1, :]: strided views with the original leading strides (no copy)."""
    k0, k1 = shard_bounds(a.shape[1], world, rank, align)
    return a[:, k0:k1], b[k0:k1, :], k0, k1


def gemm_n_sharded(a, b_local, out_local=None, bias_local=None, layout="nt", user_kwargs={}, gemm_fn: Optional[Callable] = None):
    """C[:, n0:n1] = A @ B[:, n0:n1] (+ bias[n0:n1]) on this rank. No collective."""
    if gemm_fn is None:
        from .gemm_a16w16 import gemm_a16w16 as gemm_fn
    return gemm_fn(a, b_local, out_local, bias=bias_local, user_kwargs=user_kwargs, layout=layout)


def cast_bias(src_f32: torch.Tensor, dst: torch.Tensor, bias: Optional[torch.Tensor], stream: torch.cuda.Stream) -> None:
    """dst = cast(src + bias) with the library's own kernel (one rounding, like the GEMM epilogue)."""
    ids = {torch.float32: 1, torch.bfloat16: 2, torch.float16: 3}
    rows, cols = src_f32.shape
    rc = _lib.load().b200_gemm_cast_bias(
        src_f32.data_ptr(), dst.data_ptr(), None if bias is None else bias.data_ptr(), rows, cols, ids[dst.dtype],
        0 if bias is None else ids[bias.dtype], C.c_void_p(stream.cuda_stream))
    if rc != 0:
        raise RuntimeError(f"b200_gemm_cast_bias failed ({rc}): {_lib.strerror(rc)}")


@dataclass
class KShardResult:
    out: torch.Tensor           # [sum over chunks of rows_per_rank, N]: this rank's rows, chunk after chunk
    row_ranges: list            # global [begin, end) row range of each block of `out`
    reduce_bytes: int           # fp32 bytes this rank sent into the reduce-scatter


def k_shard_row_ranges(m: int, world: int, rank: int, chunks: int) -> list[tuple[int, int]]:
    """Rows of C this rank owns after the chunked reduce-scatter: chunk c covers rows [c*mc, (c+1)*mc) and is
    split evenly over ranks, so mc must be divisible by world."""
    assert m % chunks == 0, "M must divide into equal chunks"
    mc = m // chunks
    assert mc % world == 0, "chunk rows must divide by the number of ranks"
    per = mc // world
    return [(c * mc + rank * per, c * mc + (rank + 1) * per) for c in range(chunks)]


class NcclChunkExchange:
    """Sums one chunk's fp32 partial across ranks (NCCL reduce-scatter over NVLink) and rounds this rank's rows,
    on a side stream so that it overlaps the next chunk's GEMM. CUDA only."""

    def __init__(self, device: torch.device, group, bias: Optional[torch.Tensor]):
        assert device.type == "cuda", "the K-sharded exchange runs on CUDA devices only"
        self.group = group
        self.bias = bias
        self.main = torch.cuda.current_stream(device)
        self.side = torch.cuda.Stream(device)
        self.done: dict[int, torch.cuda.Event] = {}

    def before_gemm(self, buf: int) -> None:
        ev = self.done.get(buf)
        if ev is not None:
            self.main.wait_event(ev)  # the reduce that read this partial buffer two chunks ago

    def reduce(self, buf: int, partial: torch.Tensor, reduced: torch.Tensor, dst: torch.Tensor) -> None:
        import torch.distributed as dist

        ready = torch.cuda.Event()
        ready.record(self.main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            dist.reduce_scatter_tensor(reduced, partial, op=dist.ReduceOp.SUM, group=self.group)
            cast_bias(reduced, dst, self.bias, self.side)
            ev = torch.cuda.Event()
            ev.record(self.side)
            self.done[buf] = ev

    def finish(self) -> None:
        self.main.wait_stream(self.side)


def gemm_k_sharded(a_local, b_local, out_dtype, bias=None, layout="nt", user_kwargs={}, group=None, chunks: int = 4,
                   gemm_fn: Optional[Callable] = None, exchange=None) -> KShardResult:
    """Row-sharded C = sum over ranks of A[:, k_r] @ B[k_r, :] (+ bias), rounded once to out_dtype.

    Each chunk's fp32 partial is produced on the current stream and handed to `exchange` (default: NCCL on a side
    stream); two partial buffers alternate so chunk i+1's GEMM never overwrites data the exchange still reads."""
    import torch.distributed as dist

    if gemm_fn is None:
        from .gemm_a16w16 import gemm_a16w16 as gemm_fn
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m, n = a_local.shape[0], b_local.shape[1]
    ranges = k_shard_row_ranges(m, world, rank, chunks)
    mc = m // chunks
    per = mc // world
    dev = a_local.device
    if exchange is None:
        exchange = NcclChunkExchange(dev, group, bias)
    out = torch.empty((per * chunks, n), dtype=out_dtype, device=dev)
    nbuf = min(2, chunks)
    partial = [torch.empty((mc, n), dtype=torch.float32, device=dev) for _ in range(nbuf)]
    reduced = [torch.empty((per, n), dtype=torch.float32, device=dev) for _ in range(nbuf)]
    for c in range(chunks):
        buf = c % nbuf
        exchange.before_gemm(buf)
        gemm_fn(a_local[c * mc:(c + 1) * mc], b_local, partial[buf], bias=None, user_kwargs=user_kwargs, layout=layout)
        exchange.reduce(buf, partial[buf], reduced[buf], out[c * per:(c + 1) * per])
    exchange.finish()
    return KShardResult(out=out, row_ranges=ranges, reduce_bytes=4 * m * n * (world - 1) // world)


# ------------------------------------------------------------------------------------------------------------
# Fused K-shard: the GEMM epilogue itself moves the partial sums over NVLink.
#
# Rows of C are owned in contiguous blocks (rank d owns rows [d*per, (d+1)*per)). Every rank keeps `sets` x world
# fp32 receive slots of [per, N]; slot s of rank d is written only by rank s. Rank r runs one GEMM per destination d
# — A_r[rows of d] @ B_r with fp32 output — whose `out` is slot r of rank d mapped into r's address space, so the
# epilogue's stores cross NVLink tile by tile while the tensor cores work on the next tile; destinations are visited
# in the order r+1, r+2, ..., r, so that at any moment the ranks send to different peers. One stream-ordered barrier
# later the owner sums its slots in index order (+ bias) and rounds once. With two slot sets alternating between
# calls, the barrier of call c+1 also proves that every rank has finished reading the set of call c, so one barrier
# per call is enough. No kernel ever waits on another GPU.
class PeerSlots:
    """Receive slots of the fused K-shard mode on CUDA devices: local memory exported with CUDA IPC and every peer's
    slots mapped into this process (b200_peer_export / b200_peer_open). Collective over `group`: every rank must
    construct it with the same sizes. Keep it for the life of the weights; `close()` unmaps."""

    def __init__(self, rows: int, cols: int, device: torch.device, group=None, sets: int = 2):
        import torch.distributed as dist

        assert device.type == "cuda", "peer slots live in CUDA device memory"
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.cols, self.sets, self.calls = rows, cols, sets, 0
        self.device = device
        self.local = torch.empty((sets, self.world, rows, cols), dtype=torch.float32, device=device)
        lib = _lib.load()
        mine = _lib.PeerHandle()
        with torch.cuda.device(device):
            rc = lib.b200_peer_export(self.local.data_ptr(), C.byref(mine))
        if rc != 0:
            raise RuntimeError(f"b200_peer_export failed ({rc}): {_lib.strerror(rc)}")
        blobs = [None] * self.world
        dist.all_gather_object(blobs, bytes(mine), group=group)
        self._handles, self._base = [], []
        for r, blob in enumerate(blobs):
            h = _lib.PeerHandle.from_buffer_copy(blob)
            self._handles.append(h)
            if r == self.rank:
                self._base.append(self.local.data_ptr())
                continue
            ptr = C.c_void_p()
            with torch.cuda.device(device):
                rc = lib.b200_peer_open(C.byref(h), C.byref(ptr))
            if rc != 0:
                raise RuntimeError(f"b200_peer_open of rank {r}'s slots failed ({rc}): {_lib.strerror(rc)}")
            self._base.append(ptr.value)
        dist.barrier(group=group)  # nobody stores into a peer before every mapping exists

    def next_set(self) -> int:
        s = self.calls % self.sets
        self.calls += 1
        return s

    def target(self, dest: int, set_idx: int, src: int) -> int:
        """Address, in this process, of slot `src` of set `set_idx` on rank `dest`."""
        return self._base[dest] + 4 * self.rows * self.cols * (set_idx * self.world + src)

    def local_set(self, set_idx: int) -> torch.Tensor:
        return self.local[set_idx]

    def close(self) -> None:
        lib = _lib.load()
        for r, (h, base) in enumerate(zip(self._handles, self._base)):
            if r != self.rank and base:
                with torch.cuda.device(self.device):
                    lib.b200_peer_close(C.c_void_p(base), C.byref(h))
        self._base = [0] * self.world


def reduce_slots(local_set: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor], stream: torch.cuda.Stream) -> None:
    """out = cast(sum over slots (index order) + bias) with the library's kernel."""
    ids = {torch.float32: 1, torch.bfloat16: 2, torch.float16: 3}
    n_slots, rows, cols = local_set.shape
    rc = _lib.load().b200_gemm_reduce_slots(
        local_set.data_ptr(), rows * cols, n_slots, out.data_ptr(), None if bias is None else bias.data_ptr(), rows, cols,
        ids[out.dtype], 0 if bias is None else ids[bias.dtype], C.c_void_p(stream.cuda_stream))
    if rc != 0:
        raise RuntimeError(f"b200_gemm_reduce_slots failed ({rc}): {_lib.strerror(rc)}")


def fused_send_order(world: int, rank: int) -> list[int]:
    """Destinations in the order rank `rank` serves them: its right-hand neighbours first, itself last."""
    return [(rank + j) % world for j in range(1, world + 1)]


def gemm_k_sharded_fused(a_local, b_local, out_dtype, slots, bias=None, layout="nt", user_kwargs={}, group=None, out=None,
                         gemm_into: Optional[Callable] = None, barrier: Optional[Callable] = None,
                         reduce_fn: Optional[Callable] = None) -> KShardResult:
    """Row-sharded C = sum over ranks of A[:, k_r] @ B[k_r, :] (+ bias) where the partial sums travel inside the GEMM
    epilogue (peer stores into `slots`), not in a separate collective. Rank r returns rows [r*M/world, (r+1)*M/world).

    `gemm_into(a_rows, b, target)`, `barrier()` and `reduce_fn(local_set, out, bias)` default to the CUDA path; the
    CPU tests inject their own to run the schedule with gloo ranks."""
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    m, n = a_local.shape[0], b_local.shape[1]
    assert m % world == 0, "M must divide by the number of ranks"
    per = m // world
    assert (slots.rows, slots.cols, slots.world) == (per, n, world), "slots were built for another problem"
    dev = a_local.device
    if gemm_into is None:
        from .gemm_a16w16 import gemm_a16w16_to_pointer

        def gemm_into(a_rows, b, target):
            gemm_a16w16_to_pointer(a_rows, b, target, torch.float32, user_kwargs=user_kwargs, layout=layout)
    if barrier is None:
        flag = getattr(slots, "_flag", None)
        if flag is None:
            flag = slots._flag = torch.zeros(1, dtype=torch.float32, device=dev)

        def barrier():
            # Stream-ordered on every rank: it cannot complete here before each peer has reached it, i.e. before
            # the peer's GEMMs (and their stores into this rank's slots) have finished.
            dist.all_reduce(flag, group=group)
    if reduce_fn is None:
        def reduce_fn(local_set, dst, bias_):
            reduce_slots(local_set, dst, bias_, torch.cuda.current_stream(dev))
    if out is None:
        out = torch.empty((per, n), dtype=out_dtype, device=dev)
    set_idx = slots.next_set()
    for dest in fused_send_order(world, rank):
        gemm_into(a_local[dest * per:(dest + 1) * per], b_local, slots.target(dest, set_idx, rank))
    barrier()
    reduce_fn(slots.local_set(set_idx), out, bias)
    return KShardResult(out=out, row_ranges=[(rank * per, (rank + 1) * per)], reduce_bytes=4 * per * n * (world - 1))

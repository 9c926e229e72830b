"""The allocation-free entry point, b200_gemm_a16w16_static_scratch, called straight through the C ABI.

Some hosts of this library may not allocate device memory at all (a plug-in inside an engine that owns the device
arena, a runtime that forbids cudaMalloc after start-up), so they cannot hand over a split-K workspace. For them the
library carries a fixed 16 MiB scratch array of its own. This file checks, on two calls in a row, that the result
equals what the ordinary entry point produces with a caller-provided workspace, that a plan too large for the
built-in array is refused without launching, and that no workspace pointer is needed. It is collected last so that a
`pytest -x` run has already exercised everything else.
"""
import ctypes as C

import pytest
import torch

from flydsl_examples_b200 import _lib
from flydsl_examples_b200 import gemm_a16w16 as G
from flydsl_examples_b200 import policy as P
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args_for(case: O.Case, a, b, out, bias):
    pol = P.from_user_kwargs(case.user_kwargs, case.m, case.n, case.k, case.layout)
    assert P.validate(pol, case.m, case.n, case.k, case.layout) is None
    return G._fill_args(a, b, out, bias, pol, case.layout[0] == "t", case.layout[1] == "t")


@pytest.mark.parametrize("case", [
    O.Case("split", "fp16", "tn", 130, 200, 2048, seed=61, bias_std=0.5, out_dtype="fp32", user_kwargs={"tile_n": 64, "split_k": 4}),
    O.Case("streamk", "bf16", "nt", 520, 776, 1536, seed=62, bias_std=0.5, user_kwargs={"tile_n": 128, "stream_k": True}),
    O.Case("repack", "bf16", "nn", 150, 200, 333, seed=63, bias_std=0.5, pad=3, offset=1, user_kwargs={"tile_n": 64, "split_k": 2}),
], ids=lambda c: c.name)
def test_static_scratch_matches_the_ordinary_entry_point_twice(case):
    lib = _lib.load()
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
    ref_cpu = O.reference_matmul(a_l, b_l, bias_l, case.torch_out_dtype)
    # ordinary entry point (caller-provided workspace, through the Python layer)
    want = torch.full((case.m, case.n), float("nan"), dtype=case.torch_out_dtype, device=DEV)
    G.gemm_a16w16(a, b, want, bias=bias, user_kwargs=case.user_kwargs, layout=case.layout)
    G.check_status()
    stream = torch.cuda.current_stream()
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for call in range(2):
        got = torch.full((case.m, case.n), float("nan"), dtype=case.torch_out_dtype, device=DEV)
        args = _args_for(case, a, b, got, bias)
        assert lib.b200_gemm_workspace_bytes(C.byref(args)) > 0, "the case must need scratch"
        args.workspace, args.workspace_bytes = None, 0          # the caller has none to give
        args.status = status.data_ptr()
        rc = lib.b200_gemm_a16w16_static_scratch(C.byref(args), C.c_void_p(stream.cuda_stream))
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        O.assert_close(got, want, case.k, f"{case.name} call {call} vs ordinary entry point")
        O.assert_close(got, ref_cpu, case.k, f"{case.name} call {call} vs CPU oracle")
        assert torch.equal(got, want)  # same kernel, same deterministic reduction order


def test_static_scratch_refuses_plans_beyond_its_limit():
    lib = _lib.load()
    case = O.Case("too_big", "bf16", "nt", 1024, 2048, 8192, seed=64, out_dtype="fp32", user_kwargs={"tile_n": 128, "split_k": 16})
    a = torch.zeros(case.m, case.k, dtype=torch.bfloat16, device=DEV)
    b = torch.zeros(case.n, case.k, dtype=torch.bfloat16, device=DEV).t()
    out = torch.full((case.m, case.n), 7.0, dtype=torch.float32, device=DEV)
    args = _args_for(case, a, b, out, None)
    assert lib.b200_gemm_workspace_bytes(C.byref(args)) > _lib.STATIC_SCRATCH_BYTES
    rc = lib.b200_gemm_a16w16_static_scratch(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -7 and "limit" in _lib.strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "nothing may have been launched"


def test_static_scratch_falls_back_to_the_loader_warps_for_large_unaligned_operands():
    # config 4 'nt': aligned copies of both operands would take 32.8 MB, twice the built-in array; the entry point then
    # has the kernel's loader warps fetch them, and the call needs no scratch at all
    lib = _lib.load()
    case = O.CONFIGS["c4_nt"]
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
    out = torch.full((case.m, case.n), float("nan"), dtype=torch.float32, device=DEV)
    args = _args_for(case, a, b, out, bias)
    assert lib.b200_gemm_workspace_bytes(C.byref(args)) > _lib.STATIC_SCRATCH_BYTES
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    args.status = status.data_ptr()
    rc = lib.b200_gemm_a16w16_static_scratch(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    O.assert_close(out, O.reference_matmul(a_l, b_l, bias_l, torch.float32), case.k, "c4_nt through the built-in scratch entry")


def test_static_scratch_needs_no_scratch_for_plain_tiles():
    lib = _lib.load()
    case = O.Case("plain", "bf16", "nt", 256, 512, 1024, seed=65, user_kwargs={"tile_n": 128})
    a, b, _, a_l, b_l, _ = O.build_inputs(case, device=DEV)
    out = torch.full((case.m, case.n), float("nan"), dtype=torch.bfloat16, device=DEV)
    args = _args_for(case, a, b, out, None)
    rc = lib.b200_gemm_a16w16_static_scratch(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    O.assert_close(out, O.reference_matmul(a_l, b_l, None, torch.bfloat16), case.k, "plain")


@pytest.mark.gpu
def test_library_selftest_passes_and_allocates_nothing():
    """b200_gemm_selftest: known-answer GEMMs through every tile family inside the built-in scratch array."""
    import ctypes as C

    from flydsl_examples_b200 import _lib

    lib = _lib.load()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    failed = C.c_int32(0)
    assert lib.b200_gemm_selftest(C.c_void_p(stream.cuda_stream), C.byref(failed)) == 0, f"case {failed.value}"
    assert failed.value == -1
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    assert lib.b200_gemm_selftest(C.c_void_p(stream.cuda_stream), None) == 0
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before and free_after == free_before  # no device memory was taken

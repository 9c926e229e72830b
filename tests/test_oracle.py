"""The CPU oracle against (i) the committed golden vectors produced by the reference's own `ref_func`,
(ii) the independent plain-C restatement, (iii) exact integer known-answer cases. No GPU."""
import numpy as np
import pytest
import torch

from oracle import c_ref
from oracle import oracle as O

DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def _load(golden, name):
    dt, layout, fp32 = (str(x) for x in golden[f"{name}.meta"])
    dtype = DT[dt]
    a = torch.from_numpy(golden[f"{name}.a"].copy()).view(dtype)
    b = torch.from_numpy(golden[f"{name}.b"].copy()).view(dtype)
    bias = torch.from_numpy(golden[f"{name}.bias"].copy()).view(dtype) if f"{name}.bias" in golden.files else None
    c = torch.from_numpy(golden[f"{name}.c"].copy())
    c = c if fp32 == "1" else c.view(dtype)
    return a, b, bias, c, layout


def _names(golden):
    return [str(n) for n in golden["names"]]


def test_golden_file_has_cases(golden):
    assert len(_names(golden)) >= 8


def test_ref_func_restatement_matches_golden(golden):
    # Same torch kernels as the generator: a tight bound (the summation order of a CPU mm may differ by ISA).
    for name in _names(golden):
        a, b, bias, c, _ = _load(golden, name)
        got = O.reference_ref_func(a, b, bias, c.dtype)
        assert got.dtype == c.dtype
        if c.dtype is torch.float32:
            torch.testing.assert_close(got, c, rtol=1e-5, atol=1e-4)
        else:
            # one 16-bit ulp
            torch.testing.assert_close(got.float(), c.float(), rtol=2 ** -7 if c.dtype is torch.bfloat16 else 2 ** -10, atol=1e-3)


def test_contract_oracle_within_tolerance_of_golden(golden):
    for name in _names(golden):
        a, b, bias, c, _ = _load(golden, name)
        ref = O.reference_matmul(a, b, bias, c.dtype)
        O.assert_close(ref, c, a.shape[1], name)


@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_c_restatement_matches_oracle(layout, dtype):
    case = O.Case("c", dtype, layout, 37, 53, 300, seed=7, bias_std=0.5, pad=5, offset=3)
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case)
    f32 = c_ref.gemm(a, b, bias, layout)
    f64 = c_ref.gemm(a, b, bias, layout, fp64=True)
    ref = O.reference_matmul(a_l, b_l, bias_l, torch.float32)
    torch.testing.assert_close(f32, ref, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(f64.float(), ref, rtol=1e-5, atol=1e-4)


def test_c_restatement_matches_golden(golden):
    for name in _names(golden):
        a, b, bias, c, layout = _load(golden, name)
        a_v = O.place(a, layout[0] == "t", poison=True)
        b_v = O.place(b, layout[1] == "t", poison=True)
        f32 = c_ref.gemm(a_v, b_v, bias, layout).to(c.dtype)
        O.assert_close(f32, c, a.shape[1], name)


def test_integer_known_answers():
    # Small integers: every product and partial sum is exact in fp32, so the answer is exact in any order.
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-3, 4, (17, 96), generator=g)
    b = torch.randint(-3, 4, (96, 23), generator=g)
    bias = torch.randint(-5, 6, (23,), generator=g)
    want = (a @ b + bias).float()
    for dt in (torch.bfloat16, torch.float16):
        got = O.reference_matmul(a.to(dt), b.to(dt), bias.to(dt), torch.float32)
        assert torch.equal(got, want)
        got_c = c_ref.gemm(a.to(dt).contiguous(), b.to(dt).contiguous(), bias.to(dt), "nn")
        assert torch.equal(got_c, want)
    # identity and zero
    eye = torch.eye(32, dtype=torch.bfloat16)
    x = torch.randn(32, 32).to(torch.bfloat16)
    assert torch.equal(O.reference_matmul(eye, x, None, torch.bfloat16), x)
    assert torch.equal(O.reference_matmul(torch.zeros(4, 8, dtype=torch.float16), torch.ones(8, 4, dtype=torch.float16), None, torch.float16), torch.zeros(4, 4, dtype=torch.float16))


def test_tolerance_rule():
    assert O.tolerance(1024, torch.bfloat16) == (1e-2, 1e-2)
    rtol, atol = O.tolerance(4096, torch.float32)
    assert rtol == 2e-3 and abs(atol - 4e-3) < 1e-12
    # the reference's looser rule (test_gemm_a16w16_gfx950.py:151-157)
    assert O.reference_tolerance(8192, torch.bfloat16) == (0.2, 0.2)
    r, a = O.reference_tolerance(8192, torch.float16, split_k=2, has_bias=True)
    assert r == 0.05 and abs(a - 0.05 * 2 * 1.5) < 1e-12


def test_place_layouts_and_poison():
    x = torch.arange(12, dtype=torch.float32).reshape(3, 4).to(torch.bfloat16)
    n = O.place(x, False, pad=2, offset=5)
    t = O.place(x, True, pad=2, offset=5)
    assert n.stride() == (6, 1) and t.stride() == (1, 5)
    assert n.storage_offset() == 5 and t.storage_offset() == 5
    assert torch.equal(n, x) and torch.equal(t, x)
    # bytes outside the logical matrix are NaN
    full = torch.as_strided(n, (n.untyped_storage().nbytes() // 2,), (1,), 0)
    assert torch.isnan(full.float()).sum() == full.numel() - 12


def test_configs_match_the_benchmark_list():
    c = O.CONFIGS
    assert (c["c1"].m, c["c1"].n, c["c1"].k, c["c1"].layout, c["c1"].dtype) == (256, 512, 1024, "nt", "bf16")
    assert (c["c2"].m, c["c2"].n, c["c2"].k, c["c2"].bias_std) == (2048, 4096, 4096, 0.1)
    assert (c["c3"].m, c["c3"].n, c["c3"].k, c["c3"].out_dtype, c["c3"].b_std) == (32, 384, 7168, "fp32", 0.02)
    for lay in ("nn", "nt", "tn", "tt"):
        k = c[f"c4_{lay}"]
        assert (k.m, k.n, k.k, k.pad, k.offset, k.dtype, k.out_dtype) == (1000, 3000, 4100, 64, 128, "fp16", "fp32")
    assert (c["c5"].m, c["c5"].n, c["c5"].k) == (16384, 28672, 8192)
    assert c["c3"].algorithmic_bytes == 6012928
    assert c["c2"].flops == 68719476736
    # all four C4 layouts share one oracle
    refs = [O.draw_logical(c[f"c4_{lay}"]) for lay in ("nn", "tt")]
    assert torch.equal(refs[0][0], refs[1][0]) and torch.equal(refs[0][1], refs[1][1])

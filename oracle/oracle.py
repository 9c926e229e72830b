"""CPU oracle for the A16W16 GEMM path. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this
module; the product (flydsl_examples_b200/, kernels/) never does and has no CPU path of its own.

What it restates (xytpai/flydsl-examples):
  * ref_func        test_gemm_a16w16_gfx950.py:82-94   torch.mm / torch.addmm reference of the reference's tests
  * create_inputs   test_gemm_a16w16_gfx950.py:47-73   layout-shaped operands ('t' = allocate transposed, view back)
  * create_outputs  test_gemm_a16w16_gfx950.py:76-79   outputs pre-filled with randn so stale data is caught
  * get_tol         test_gemm_a16w16_gfx950.py:151-157 the reference's (loose) tolerance rule
  * kernel numerics kernels/gemm_a16w16_gfx950.py:613-620 (fp32 accumulate), :541-550 (bias joins in fp32)

The bar used here is the stricter one of the build contract: an fp32 `torch.matmul` on up-cast inputs plus fp32
bias, cast ONCE to the output dtype; rtol 1e-2 / atol 1e-2*sqrt(K/1024) for 16-bit outputs, rtol 2e-3 /
atol 2e-3*sqrt(K/1024) for fp32 outputs (the contract names no fp32 atol; this one is ours), the same bound for
split-K. The reference's 16-bit staging, 16-bit slice-K sums and packed 16-bit atomics
(kernels/gemm_a16w16_gfx950.py:660-661, :689-694, :356-373) are deliberately not restated.

Pinning: the reference stores no golden vectors and cannot run here (it needs FlyDSL + a gfx950 GPU). This oracle
is pinned (tests/test_oracle.py) against (i) an independent plain-C restatement (oracle/gemm_ref.c: naive fp32 and
fp64 triple loops), (ii) the reference's own `ref_func` semantics on the committed fixtures in tests/golden/, and
(iii) exact integer-valued known-answer cases.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def reference_matmul(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """fp32-accumulated A[M,K] @ B[K,N] (+ bias[N]) on CPU, one cast to out_dtype."""
    a32 = a.detach().to("cpu", torch.float32)
    b32 = b.detach().to("cpu", torch.float32)
    ref = torch.matmul(a32, b32)
    if bias is not None:
        ref += bias.detach().to("cpu", torch.float32)
    return ref.to(out_dtype)


def reference_ref_func(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """The reference test's own oracle (test_gemm_a16w16_gfx950.py:82-94): same-dtype mm/addmm for 16-bit
    outputs, up-cast mm/addmm for fp32 outputs."""
    a, b = a.detach().cpu(), b.detach().cpu()
    bias = None if bias is None else bias.detach().cpu()
    if out_dtype == a.dtype:
        return torch.mm(a, b) if bias is None else torch.addmm(bias, a, b)
    if bias is None:
        return torch.mm(a.float(), b.float())
    return torch.addmm(bias.float(), a.float(), b.float())


def tolerance(k: int, out_dtype: torch.dtype) -> tuple[float, float]:
    """(rtol, atol) of the build contract."""
    scale = math.sqrt(max(k, 1) / 1024.0)
    if out_dtype is torch.float32:
        return 2e-3, 2e-3 * scale
    return 1e-2, 1e-2 * scale


def reference_tolerance(k: int, dtype: torch.dtype, split_k: int = 1, k_waves: int = 1, has_bias: bool = False) -> tuple[float, float]:
    """(rtol, atol) of the reference's tests (test_gemm_a16w16_gfx950.py:151-157); looser than `tolerance`."""
    k_scale = math.sqrt(k / 8192.0) * split_k * k_waves
    atol_scale = 1.5 if has_bias else 1.0
    if dtype is torch.bfloat16:
        return 2e-1, 2e-1 * k_scale * atol_scale
    return 5e-2, 5e-2 * k_scale * atol_scale


def compare(got: torch.Tensor, ref: torch.Tensor, k: int) -> dict:
    """Error summary of `got` against `ref` under `tolerance`; never raises."""
    rtol, atol = tolerance(k, ref.dtype)
    g = got.detach().to("cpu", torch.float32)
    r = ref.detach().to("cpu", torch.float32)
    finite = bool(torch.isfinite(g).all())
    diff = (g - r).abs()
    bound = atol + rtol * r.abs()
    bad = int((~(diff <= bound)).sum())
    big = r.abs() > 0.01
    max_rel = float((diff[big] / r.abs()[big]).max()) if bool(big.any()) else 0.0
    return {
        "ok": finite and bad == 0,
        "finite": finite,
        "mismatches": bad,
        "max_abs": float(diff.max()) if diff.numel() else 0.0,
        "max_rel_over_0.01": max_rel,
        "rtol": rtol,
        "atol": atol,
    }


def assert_close(got: torch.Tensor, ref: torch.Tensor, k: int, what: str = "") -> dict:
    res = compare(got, ref, k)
    assert got.dtype == ref.dtype, f"{what}: dtype {got.dtype} != {ref.dtype}"
    assert tuple(got.shape) == tuple(ref.shape), f"{what}: shape {tuple(got.shape)} != {tuple(ref.shape)}"
    assert res["ok"], f"{what}: {res}"
    return res


# ----------------------------------------------------------------------------------------------------------------
# Seeded synthetic inputs. Everything is drawn on the CPU from one torch.Generator so the oracle and the GPU see the
# same bits; operands are then *placed* into layout-shaped (optionally padded / offset / NaN-poisoned) storage.

@dataclass
class Case:
    name: str
    dtype: str
    layout: str
    m: int
    n: int
    k: int
    seed: int
    a_std: float = 1.0
    b_std: float = 1.0
    bias_std: Optional[float] = None  # None = no bias
    out_dtype: Optional[str] = None   # None = input dtype
    pad: int = 0                      # extra elements on every operand's leading stride
    offset: int = 0                   # storage offset (elements) of every operand inside a larger buffer
    user_kwargs: dict = field(default_factory=dict)

    @property
    def torch_dtype(self) -> torch.dtype:
        return DTYPES[self.dtype]

    @property
    def torch_out_dtype(self) -> torch.dtype:
        return DTYPES[self.out_dtype or self.dtype]

    @property
    def flops(self) -> int:
        return 2 * self.m * self.n * self.k

    @property
    def algorithmic_bytes(self) -> int:
        out_es = 4 if (self.out_dtype or self.dtype) == "fp32" else 2
        return 2 * (self.m * self.k + self.k * self.n) + out_es * self.m * self.n + (2 * self.n if self.bias_std is not None else 0)


# The five benchmark configurations (BASELINE.json "configs", in order).
CONFIGS = {
    "c1": Case("c1", "bf16", "nt", 256, 512, 1024, seed=0),
    "c2": Case("c2", "bf16", "nt", 2048, 4096, 4096, seed=1, bias_std=0.1),
    "c3": Case("c3", "bf16", "nt", 32, 384, 7168, seed=2, b_std=0.02, out_dtype="fp32"),
    "c4_nn": Case("c4_nn", "fp16", "nn", 1000, 3000, 4100, seed=3, bias_std=0.1, out_dtype="fp32", pad=64, offset=128),
    "c4_nt": Case("c4_nt", "fp16", "nt", 1000, 3000, 4100, seed=3, bias_std=0.1, out_dtype="fp32", pad=64, offset=128),
    "c4_tn": Case("c4_tn", "fp16", "tn", 1000, 3000, 4100, seed=3, bias_std=0.1, out_dtype="fp32", pad=64, offset=128),
    "c4_tt": Case("c4_tt", "fp16", "tt", 1000, 3000, 4100, seed=3, bias_std=0.1, out_dtype="fp32", pad=64, offset=128),
    "c5": Case("c5", "bf16", "nt", 16384, 28672, 8192, seed=4, a_std=0.02, b_std=0.02),
}


def draw_logical(case: Case) -> tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Contiguous logical A[M,K], B[K,N], bias[N] in the input dtype (CPU). Draw order: A, then B *as stored*
    ([N,K] for a 't' B, [K,N] for an 'n' B — except that padded/offset sweeps draw B as [K,N] once so all four
    layouts share one oracle), then bias."""
    g = torch.Generator("cpu").manual_seed(case.seed)
    dt = case.torch_dtype
    a = (torch.randn(case.m, case.k, generator=g, dtype=torch.float32) * case.a_std).to(dt)
    if case.layout[1] == "t" and case.pad == 0 and case.offset == 0:
        b = (torch.randn(case.n, case.k, generator=g, dtype=torch.float32) * case.b_std).to(dt).t()
    else:
        b = (torch.randn(case.k, case.n, generator=g, dtype=torch.float32) * case.b_std).to(dt)
    bias = None
    if case.bias_std is not None:
        bias = (torch.randn(case.n, generator=g, dtype=torch.float32) * case.bias_std).to(dt)
    return a, b, bias


def place(logical: torch.Tensor, transposed: bool, pad: int = 0, offset: int = 0, device="cpu", poison: bool = True) -> torch.Tensor:
    """Return a [rows, cols] view with the given layout living inside a larger 1-D buffer:
    'n' -> strides (cols+pad, 1); 't' -> strides (1, rows+pad); storage offset `offset` elements.
    Padding and the bytes around the view are NaN so a kernel that reads outside the logical matrix is caught."""
    rows, cols = logical.shape
    lead_extent = rows if transposed else cols
    other = cols if transposed else rows
    ld = lead_extent + pad
    total = offset + other * ld + 64
    buf = torch.full((total,), float("nan") if poison else 0.0, dtype=logical.dtype, device=device)
    if transposed:
        view = torch.as_strided(buf, (rows, cols), (1, ld), offset)
    else:
        view = torch.as_strided(buf, (rows, cols), (ld, 1), offset)
    view.copy_(logical.to(device))
    return view


def build_inputs(case: Case, device="cpu"):
    """(a_view, b_view, bias, a_logical_cpu, b_logical_cpu, bias_cpu) for a case."""
    a, b, bias = draw_logical(case)
    a_v = place(a, case.layout[0] == "t", case.pad, case.offset, device)
    b_v = place(b, case.layout[1] == "t", case.pad, case.offset, device)
    bias_v = None if bias is None else bias.to(device)
    return a_v, b_v, bias_v, a, b, bias


def expected(case: Case) -> torch.Tensor:
    a, b, bias = draw_logical(case)
    return reference_matmul(a, b, bias, case.torch_out_dtype)

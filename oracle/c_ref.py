"""ctypes access to oracle/gemm_ref.c (plain-C fp32 / fp64 restatement). TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
LIB = HERE / "libgemm_ref.so"
_lib = None


def build() -> Path:
    src = HERE / "gemm_ref.c"
    if not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "libgemm_ref.so"], check=True, capture_output=True)
    return LIB


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB))
        for name, out_t in (("gemm_ref_f32", C.c_float), ("gemm_ref_f64", C.c_double)):
            fn = getattr(_lib, name)
            fn.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_void_p,
                           C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
            fn.restype = None
    return _lib


def gemm(a: torch.Tensor, b: torch.Tensor, bias, layout: str, fp64: bool = False) -> torch.Tensor:
    """a: [M,K] view, b: [K,N] view (CPU, bf16/fp16) with the strides `layout` promises. Returns fp32/fp64 [M,N]."""
    assert a.device.type == "cpu" and b.device.type == "cpu"
    a_t, b_t = layout[0] == "t", layout[1] == "t"
    m, k = a.shape
    n = b.shape[1]
    lda = a.stride(1) if a_t else a.stride(0)
    ldb = b.stride(1) if b_t else b.stride(0)
    assert (a.stride(0) if a_t else a.stride(1)) == 1 and (b.stride(0) if b_t else b.stride(1)) == 1
    dt = 2 if a.dtype is torch.bfloat16 else 3
    out = torch.empty(m, n, dtype=torch.float64 if fp64 else torch.float32)
    fn = load().gemm_ref_f64 if fp64 else load().gemm_ref_f32
    fn(a.data_ptr(), lda, int(a_t), b.data_ptr(), ldb, int(b_t), None if bias is None else bias.data_ptr(),
       m, n, k, dt, out.data_ptr())
    return out

"""`torch.library` registration of the GEMM so that it can sit inside `torch.compile`d graphs and CUDA-graph
captured decode loops as an opaque operator (no tracing into ctypes).

Plays the role the reference's benchmark gives to a "FLYDSL" inductor backend living in a PyTorch fork
(torch_benchmark.py:32-49, :62-77): there the compiler picks the kernel as a GEMM template; here the compiled graph
simply calls `torch.ops.b200.gemm_a16w16`. Importing this module registers the operator.

    import flydsl_examples_b200.torch_op            # registers torch.ops.b200.gemm_a16w16
    y = torch.ops.b200.gemm_a16w16(a, b, bias, "nt", None)
"""
from __future__ import annotations

from typing import Optional

import torch

from .gemm_a16w16 import gemm_a16w16 as _gemm

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


@torch.library.custom_op("b200::gemm_a16w16", mutates_args=())
def gemm_a16w16_op(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], layout: str,
                   out_dtype: Optional[str]) -> torch.Tensor:
    """C = A @ B (+ bias). `layout` as in gemm_a16w16; `out_dtype` is None (input dtype), "fp32", "bf16" or "fp16"."""
    dt = None if out_dtype is None else _DTYPES[out_dtype]
    return _gemm(a, b, None, bias=bias, layout=layout, out_dtype=dt)


@gemm_a16w16_op.register_fake
def _(a, b, bias, layout, out_dtype):
    if layout.lower() not in ("nn", "nt", "tn", "tt"):
        raise ValueError(f"unsupported GEMM layout: {layout!r}")
    torch._check(a.dim() == 2 and b.dim() == 2)
    torch._check(a.shape[1] == b.shape[0])
    dt = a.dtype if out_dtype is None else _DTYPES[out_dtype]
    return a.new_empty((a.shape[0], b.shape[1]), dtype=dt)

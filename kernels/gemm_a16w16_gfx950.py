"""Drop-in import path of the reference's public op (kernels/gemm_a16w16_gfx950.py:1288 in
xytpai/flydsl-examples). The names its callers import (its tests, gemm_tune.py:19-24, the README quick start)
resolve here to the B200 implementation in flydsl_examples_b200."""
from flydsl_examples_b200.gemm_a16w16 import (  # noqa: F401
    GEMM_A16W16_DTYPE_BF16,
    GEMM_A16W16_DTYPE_FP16,
    GEMM_A16W16_DTYPE_FP32,
    gemm_a16w16,
    make_gemm_a16w16_param_and_validate,
)

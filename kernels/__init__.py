"""Import path kept from xytpai/flydsl-examples (`kernels.gemm_a16w16_gfx950`); the code lives in flydsl_examples_b200."""

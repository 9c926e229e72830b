"""Constants the reference's callers import from kernels/gemm_a16w16_gfx950_utils.py (:14-16)."""
from flydsl_examples_b200.gemm_a16w16 import DMA_BYTES

# 16-byte transfer granule: the reference's direct-to-LDS DMA width, and TMA's alignment granule on sm_100a.
GFX950_DMA_BYTES = DMA_BYTES

/* Plain-C restatement of the A16W16 GEMM arithmetic. TEST INFRASTRUCTURE ONLY (checker, never shipped or timed as
 * the product). Independent of torch: used to pin oracle/oracle.py and as the single-thread "port" CPU baseline.
 *
 * Follows xytpai/flydsl-examples:
 *   kernels/gemm_a16w16_gfx950.py:613-620   16-bit products accumulated in fp32 (MFMA f32 accumulate)
 *   kernels/gemm_a16w16_gfx950.py:541-550   bias[n] joins the accumulator as fp32
 *   kernels/gemm_a16w16_gfx950.py:684       only the logical M x N region is written
 *   kernels/gemm_a16w16_gfx950.py:1298-1306 a layout letter only says which dimension is contiguous
 * Not restated on purpose: the reference's 16-bit staging / slice-K sums / 16-bit atomics (:660-661, :689-694,
 * :356-373); the bar is one rounding from an fp32 (or, for gemm_ref_f64, exact-enough fp64) sum.
 */
#include <stdint.h>
#include <string.h>

#define DT_BF16 2
#define DT_FP16 3

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static float fp16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else { /* subnormal: renormalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static float load16(const uint16_t* p, int dtype) { return dtype == DT_BF16 ? bf16_to_f32(*p) : fp16_to_f32(*p); }

/* A is logical [M,K]: element (i,l) at a[i*lda + l] when a_trans == 0, a[l*lda + i] when 1.
 * B is logical [K,N]: element (l,j) at b[l*ldb + j] when b_trans == 0, b[j*ldb + l] when 1.
 * out is row-major fp32 [M,N]. Accumulation order: l = 0..K-1, sequential, in fp32. */
void gemm_ref_f32(const uint16_t* a, int64_t lda, int a_trans, const uint16_t* b, int64_t ldb, int b_trans,
                  const uint16_t* bias, int64_t m, int64_t n, int64_t k, int dtype, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.f;
      for (int64_t l = 0; l < k; ++l) {
        const float x = load16(a_trans ? a + l * lda + i : a + i * lda + l, dtype);
        const float y = load16(b_trans ? b + j * ldb + l : b + l * ldb + j, dtype);
        acc += x * y;
      }
      if (bias) acc += load16(bias + j, dtype);
      out[i * n + j] = acc;
    }
  }
}

/* Same with an fp64 accumulator (products of two 16-bit values are exact in fp64): the "true" value up to one
 * final rounding, used to bound the fp32 paths. */
void gemm_ref_f64(const uint16_t* a, int64_t lda, int a_trans, const uint16_t* b, int64_t ldb, int b_trans,
                  const uint16_t* bias, int64_t m, int64_t n, int64_t k, int dtype, double* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double acc = 0.0;
      for (int64_t l = 0; l < k; ++l) {
        const double x = load16(a_trans ? a + l * lda + i : a + i * lda + l, dtype);
        const double y = load16(b_trans ? b + j * ldb + l : b + l * ldb + j, dtype);
        acc += x * y;
      }
      if (bias) acc += load16(bias + j, dtype);
      out[i * n + j] = acc;
    }
  }
}

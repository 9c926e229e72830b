// The small kernels of libb200_gemm.so besides the GEMM itself: the bounded-wait self-test, the aligned repack of
// operands that neither TMA nor the in-kernel loader can take, the cast/bias and slot-reduction kernels of the
// K-sharded multi-GPU modes, and the helpers of b200_gemm_selftest. Included by one translation unit only.
#pragma once
#include "gemm_kernel.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------------------
// The bounded wait on its own: one thread waits on a barrier that nobody signals; the wait gives up after
// `limit_ns` and the thread reports it in the 4-word status block like the GEMM roles do (role 9 = this test).
__global__ void wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    const bool completed = mbar_wait(smem_u32(&bar), 0u, &abort_flag, limit_ns);
    if (!completed && atomicCAS(status, 0, 1) == 0) {
      status[1] = (int)blockIdx.x;
      status[2] = 9;
      status[3] = -1;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Aligned repack: copies a 16-bit matrix whose base or pitch is not 16-byte aligned (TMA cannot describe it)
// into a scratch image with a pitch that is a multiple of 8 elements. rows x cols, cols contiguous.
// The reference rejects such operands (kernels/gemm_a16w16_gfx950.py:1322-1372); this path accepts them.
__device__ __forceinline__ void repack_rows_body(const uint16_t* __restrict__ src, long long src_ld, uint16_t* __restrict__ dst,
                                                 long long dst_ld, int rows, int cols, int block, int nblocks) {
  const int chunks = (cols + 7) >> 3;
  const long long total = (long long)rows * chunks;
  for (long long i = block * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)nblocks * blockDim.x) {
    const int r = (int)(i / chunks);
    const int c0 = (int)(i - (long long)r * chunks) << 3;
    const uint16_t* s = src + (long long)r * src_ld + c0;
    uint32_t w[4] = {0, 0, 0, 0};
    const int n = min(8, cols - c0);
    if (n == 8 && (reinterpret_cast<uintptr_t>(s) & 7) == 0) {
      const uint2 a = __ldg(reinterpret_cast<const uint2*>(s));
      const uint2 b = __ldg(reinterpret_cast<const uint2*>(s) + 1);
      w[0] = a.x, w[1] = a.y, w[2] = b.x, w[3] = b.y;
    } else if (n == 8 && (reinterpret_cast<uintptr_t>(s) & 3) == 0) {
      const uint32_t* s4 = reinterpret_cast<const uint32_t*>(s);
      w[0] = __ldg(s4), w[1] = __ldg(s4 + 1), w[2] = __ldg(s4 + 2), w[3] = __ldg(s4 + 3);
    } else {
      for (int j = 0; j < n; ++j) w[j >> 1] |= uint32_t(__ldg(s + j)) << ((j & 1) * 16);
    }
    *reinterpret_cast<uint4*>(dst + (long long)r * dst_ld + c0) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// One launch repacks up to two operands: blocks [0, blocks0) take the first job, the rest the second.
__global__ void repack_rows_kernel(const uint16_t* __restrict__ src0, long long src_ld0, uint16_t* __restrict__ dst0,
                                   long long dst_ld0, int rows0, int cols0, int blocks0, const uint16_t* __restrict__ src1,
                                   long long src_ld1, uint16_t* __restrict__ dst1, long long dst_ld1, int rows1, int cols1) {
  // The GEMM that follows is launched as a programmatic dependent: it may set up (barriers, TMEM, descriptors) while
  // this grid copies; it reads the images only after its own wait for this grid's completion.
  grid_launch_dependents();
  if ((int)blockIdx.x < blocks0)
    repack_rows_body(src0, src_ld0, dst0, dst_ld0, rows0, cols0, (int)blockIdx.x, blocks0);
  else
    repack_rows_body(src1, src_ld1, dst1, dst_ld1, rows1, cols1, (int)blockIdx.x - blocks0, (int)gridDim.x - blocks0);
}

// ---------------------------------------------------------------------------------------------------------
// out[r, c] = bias[c] (or 0) for an fp32 matrix with row stride ldo: what C must hold before a GEMM whose K-parallel
// units add their partial sums into it (atomic split mode). cols % 4 == 0 and 16-byte aligned rows (the same
// condition that lets the GEMM reach C through TMA).
__global__ void init_out_rows_kernel(float* __restrict__ out, long long ldo, int rows, int cols, const void* __restrict__ bias,
                                     int bias_dtype) {
  grid_launch_dependents();  // the GEMM behind may set up meanwhile; it touches C only after this grid has completed
  const int c4 = cols >> 2;
  const long long total = (long long)rows * c4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / c4), c = (int)(i - (long long)r * c4) << 2;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias != nullptr) {
      x.x = load_in_as_float(bias, c, bias_dtype), x.y = load_in_as_float(bias, c + 1, bias_dtype);
      x.z = load_in_as_float(bias, c + 2, bias_dtype), x.w = load_in_as_float(bias, c + 3, bias_dtype);
    }
    *reinterpret_cast<float4*>(out + (long long)r * ldo + c) = x;
  }
}

// ---------------------------------------------------------------------------------------------------------
// fp32 [rows, cols] (+ bias[cols] in `bias_dtype`) -> 16-bit or fp32 [rows, cols]; both row-major contiguous.
// Final step of the K-sharded multi-GPU mode: the fp32 partial sums have been reduced across GPUs and are
// rounded once here, exactly like the single-GPU epilogue.
__global__ void cast_bias_rows_kernel(const float* __restrict__ in, void* __restrict__ out, const void* __restrict__ bias,
                                      long long rows, int cols, int out_dtype, int bias_dtype) {
  const long long total4 = rows * (long long)cols / 4;  // cols % 4 == 0 is checked by the host
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    float4 x = __ldcs(reinterpret_cast<const float4*>(in) + i);
    if (bias != nullptr) {
      const int c = (int)((i * 4) % cols);
      x.x += load_in_as_float(bias, c, bias_dtype);
      x.y += load_in_as_float(bias, c + 1, bias_dtype);
      x.z += load_in_as_float(bias, c + 2, bias_dtype);
      x.w += load_in_as_float(bias, c + 3, bias_dtype);
    }
    if (out_dtype == 1) {
      reinterpret_cast<float4*>(out)[i] = x;
    } else if (out_dtype == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
      __half2 lo = __floats2half2_rn(x.x, x.y), hi = __floats2half2_rn(x.z, x.w);
      reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// out[rows, cols] = cast(sum over s < n_slots of slots[s * slot_stride + ...] + bias[cols]); every slot is a
// row-major contiguous fp32 [rows, cols] image. Owner-side reduction of the fused K-sharded multi-GPU mode: slot s
// was filled over NVLink by rank s's GEMM epilogue (peer stores), slot `own` by this GPU's GEMM. The slots are
// summed in index order, so every rank's result is bitwise independent of arrival order.
__global__ void reduce_slots_kernel(const float* __restrict__ slots, long long slot_stride, int n_slots,
                                    void* __restrict__ out, const void* __restrict__ bias, long long rows, int cols,
                                    int out_dtype, int bias_dtype) {
  const long long total4 = rows * (long long)cols / 4;  // cols % 4 == 0 is checked by the host
  const long long stride4 = slot_stride / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    const float4* src = reinterpret_cast<const float4*>(slots) + i;
    float4 x = __ldcs(src);
    int s = 1;
    for (; s + 4 <= n_slots; s += 4) {  // four independent loads in flight per thread
      const float4 a = __ldcs(src + s * stride4), b = __ldcs(src + (s + 1) * stride4);
      const float4 c = __ldcs(src + (s + 2) * stride4), d = __ldcs(src + (s + 3) * stride4);
      x.x = (((x.x + a.x) + b.x) + c.x) + d.x, x.y = (((x.y + a.y) + b.y) + c.y) + d.y;
      x.z = (((x.z + a.z) + b.z) + c.z) + d.z, x.w = (((x.w + a.w) + b.w) + c.w) + d.w;
    }
    for (; s < n_slots; ++s) {
      const float4 a = __ldcs(src + s * stride4);
      x.x += a.x, x.y += a.y, x.z += a.z, x.w += a.w;
    }
    if (bias != nullptr) {
      const int c = (int)((i * 4) % cols);
      x.x += load_in_as_float(bias, c, bias_dtype);
      x.y += load_in_as_float(bias, c + 1, bias_dtype);
      x.z += load_in_as_float(bias, c + 2, bias_dtype);
      x.w += load_in_as_float(bias, c + 3, bias_dtype);
    }
    if (out_dtype == 1) {
      reinterpret_cast<float4*>(out)[i] = x;
    } else if (out_dtype == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
      __half2 lo = __floats2half2_rn(x.x, x.y), hi = __floats2half2_rn(x.z, x.w);
      reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Self-test helpers (b200_gemm_selftest): small-integer operands, an exact CUDA-core reference, an exact compare.
__device__ __forceinline__ uint16_t selftest_encode_float(float v, int dtype) {
  if (dtype == 2) {
    __nv_bfloat16 h = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&h);
  }
  __half h = __float2half_rn(v);
  return *reinterpret_cast<uint16_t*>(&h);
}
__device__ __forceinline__ uint16_t selftest_encode(int v, int dtype) { return selftest_encode_float((float)v, dtype); }

// dst[r * ld + c] = ((r * 131 + c * 71 + seed) % 5) - 2 for r < rows, c < cols, as bf16 / fp16.
__global__ void selftest_fill_kernel(uint16_t* __restrict__ dst, int rows, int cols, long long ld, int dtype, int seed) {
  const long long total = (long long)rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
    dst[(long long)r * ld + c] = selftest_encode(((r * 131 + c * 71 + seed) % 5) - 2, dtype);
  }
}

// ref[m * N + n] = sum_k A[m,k] * B[k,n] + bias[n] in fp32 (exact for the small integers above).
__global__ void selftest_ref_kernel(const uint16_t* __restrict__ a, long long lda, int a_trans, const uint16_t* __restrict__ b,
                                    long long ldb, int b_trans, const uint16_t* __restrict__ bias, int M, int N, int K,
                                    int dtype, float* __restrict__ ref) {
  const long long total = (long long)M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / N), n = (int)(i - (long long)m * N);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const float x = load_in_as_float(a, a_trans ? (long long)k * lda + m : (long long)m * lda + k, dtype);
      const float y = load_in_as_float(b, b_trans ? (long long)n * ldb + k : (long long)k * ldb + n, dtype);
      acc += x * y;
    }
    if (bias != nullptr) acc += load_in_as_float(bias, n, dtype);
    ref[i] = acc;
  }
}

// Counts elements of out (fp32, bf16 or fp16; row-major contiguous) that differ from the reference rounded the same way.
__global__ void selftest_compare_kernel(const void* __restrict__ out, int out_dtype, const float* __restrict__ ref,
                                        long long total, int* __restrict__ mismatches) {
  int bad = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    if (out_dtype == 1) {
      bad += reinterpret_cast<const float*>(out)[i] != ref[i];
    } else {
      bad += reinterpret_cast<const uint16_t*>(out)[i] != selftest_encode_float(ref[i], out_dtype);
    }
  }
  if (bad) atomicAdd(mismatches, bad);
}

}  // namespace b200

// Persistent, warp-specialised A16W16 GEMM for sm_100a.
//
//   D[P,Q] = U[P,K] * V[Q,K]^T        U = the operand that sits on the 128-row MMA axis (TMEM lanes)
//                                      V = the operand that sits on the MMA N axis (TMEM columns)
// The host maps (A,B) -> (U,V) normally and (B,A) -> (U,V) for swap_ab; the epilogue then writes D or D^T.
// Either operand may be K-contiguous ("K-major") or P/Q-contiguous ("MN-major"): that only changes how the
// host encodes the tensor map, how many 64-wide TMA boxes one stage takes, and two descriptor fields.
//
// Roles (192 threads): warp 0 = TMA producer (one elected lane), warp 1 = TMEM owner + MMA issuer (one lane),
// warps 2..5 = epilogue (warp w owns TMEM lanes 32*(w%4)..+31). The LOADER variants have two more warps (6, 7)
// that fetch K-contiguous operands TMA cannot describe (base or pitch not a multiple of 16 bytes) with per-thread
// cp.async copies, writing the very 128-byte-swizzled image a TMA box would have left. The accumulator is double-buffered in TMEM so the
// epilogue of one unit overlaps the main loop of the next. A work unit is (output tile, K-slice); CTA b walks
// units b, b+grid, b+2*grid, ...
//
// Covers the reference's gemm_a16w16_gfx950_kernel / gemm_a16w16_hti_gfx950_kernel
// (kernels/gemm_a16w16_gfx950.py:378-705, :708-1142), async_load_to_lds (:263-322), the bias/cast/store
// epilogue (:660-703, :325-375), SplitKProtocol (kernels/gemm_a16w16_gfx950_utils.py:100-299) and
// BlockSwizzle (kernels/gemm_a16w16_gfx950_utils.py:65-97).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace b200 {

constexpr int kTileP = 128;  // rows of U per CTA tile (MMA M)
constexpr int kBoxK = 64;    // K elements per TMA box = one 128-byte swizzle span of 16-bit data
constexpr int kUmmaK = 16;   // K elements per tcgen05.mma kind::f16
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kLoaderThreads = 64;                       // warps 6 and 7 of a LOADER variant (256 threads: 255 registers each)
constexpr int kThreadsLoader = kThreads + kLoaderThreads;
constexpr int kUBoxBytes = kTileP * kBoxK * 2;  // 16 KB: the 128 U rows of one 64-deep K box

struct alignas(64) GemmParams {
  CUtensorMap tmap_u;
  CUtensorMap tmap_v;
  CUtensorMap tmap_out;  // output, box = 32 rows x 128 bytes (valid when tma_store != 0)
  void* out;
  const void* bias;
  float* partials;  // [tile][slice][chunk][128][CW] fp32
  int* tickets;     // [tile]
  int* status;      // int32[4] or null
  unsigned long long* trace;  // optional timeline: [cta][role 0..3][item 0..15][4] stamps / counters, or null
  int trace_detail;           // 1: also count cycles per K block in the MMA warp (slows the kernel down)
  long long ldo;    // output row stride (elements)
  int P, Q, K;
  int tiles_p, tiles_q, num_tiles;
  int kb_total;  // ceil(K / TK): K blocks of one pipeline stage each
  int split_k;
  int cluster_split;  // > 1: the split_k CTAs of a tile form one thread-block cluster and reduce through DSMEM
  int num_units;
  int sk_tiles;     // stream-K: the first sk_tiles tiles are cut into equal K spans over all CTAs (0 = off)
  int sk_slots;     // stream-K: partial-tile slots reserved per tile (upper bound of contributors)
  int group_p;      // grouped rasterisation over tile rows of P (0 = off)
  int swap_out;     // 1: D^T is written (out[q*ldo + p]); bias indexed by p
  int tma_store;    // 1: finished tiles leave through swizzled staging smem and TMA stores (needs 16-byte aligned C rows)
  int atomic_out;   // 1: a partial unit adds its fp32 sums straight into `out` with TMA reduce-add (no workspace, no tickets);
                    //    `out` (fp32) holds the bias, or zero, before the kernel starts, and whole tiles overwrite it
  int out_dtype;    // 1 fp32, 2 bf16, 3 fp16
  int in_dtype;     // 2 bf16, 3 fp16
  int u_mn_major;   // 1: U is P-contiguous, loaded as two [64 P x 64 K] boxes
  int v_mn_major;   // 1: V is Q-contiguous, loaded as TILE_Q/64 boxes
  uint32_t idesc;   // tcgen05 instruction descriptor
  uint32_t idesc2;  // 512-column variant: descriptor of the second MMA of a K step (N = tile_q - 256)
  int tile_q;       // 512-column variant: columns of one tile, 288..512 in steps of 32 (the other variants use TILE_Q)
  uint32_t u_desc_hi, u_desc_lo;  // smem matrix descriptor without the start address
  uint32_t v_desc_hi, v_desc_lo;
  uint32_t u_kstep, v_kstep;  // start-address increment (16-byte units) per K=16 MMA inside a stage
  unsigned long long wait_limit_ns;  // time limit of every wait inside the kernel
  // LOADER variants only: operands fetched by the loader warps instead of TMA (K-contiguous rows, 8-byte aligned)
  const void* u_src;
  const void* v_src;
  long long u_pitch, v_pitch;  // bytes between consecutive rows
  int u_cp, v_cp;              // 1: this operand comes through cp.async
  uint32_t tma_tx_bytes;       // bytes per stage that TMA still delivers (both CTAs of a pair together)
};

// One piece of work of a CTA: K blocks kb0, kb0+kstep, ... (kbn of them) of output tile (tp, tq). When `partial`, the fp32 result goes to
// slot `slot` of the workspace and the last of `n_contrib` contributors (ticket) reduces slots slot0..slot0+n_contrib-1.
struct Unit {
  int tile, tp, tq, kb0, kbn, kstep;
  int partial, slot, slot0, n_contrib;
};

__device__ __forceinline__ void raster_tile(const GemmParams& p, int tile, int& tp, int& tq) {
  if (p.group_p > 0) {
    const int per_group = p.group_p * p.tiles_q;
    const int g = tile / per_group;
    const int first = g * p.group_p;
    const int rows = min(p.tiles_p - first, p.group_p);
    const int r = tile - g * per_group;
    tp = first + r % rows;
    tq = r / rows;
  } else {
    tp = tile / p.tiles_q;
    tq = tile - tp * p.tiles_q;
  }
}

// Walks the work of one CTA (or CTA pair); all three roles run the same walk.
//   split-K / data-parallel (sk_tiles == 0): units u = cta, cta+grid, ... ; unit = (tile, K slice).
//   stream-K (sk_tiles > 0): first this CTA's equal share of the K blocks of tiles [0, sk_tiles) (a contiguous span
//   that may cross tile boundaries), then whole tiles sk_tiles + cta, sk_tiles + cta + grid, ...
struct WorkIter {
  long long sk_cur, sk_end, sk_total;
  int next_u, me, count;
  // `me` of `count`: this CTA among the CTAs of the grid, or this CTA pair among the pairs.
  __device__ __forceinline__ void init(const GemmParams& p, int me_, int count_) {
    me = me_, count = count_;
    sk_total = (long long)p.sk_tiles * p.kb_total;
    sk_cur = sk_total * me / count;
    sk_end = sk_total * (me + 1) / count;
    next_u = p.sk_tiles > 0 ? p.sk_tiles + me : me;
  }
  // Walker that owns stream-K iteration x: the largest b with floor(b * total / count) <= x.
  __device__ __forceinline__ int owner(long long x) const {
    return (int)(((x + 1) * count + sk_total - 1) / sk_total) - 1;
  }
  // After next(): does this walker have another unit to come?
  __device__ __forceinline__ bool more(const GemmParams& p) const {
    if (sk_cur < sk_end) return true;
    return next_u < (p.sk_tiles > 0 ? p.num_tiles : p.num_units);
  }
  __device__ __forceinline__ bool next(const GemmParams& p, Unit& w) {
    if (sk_cur < sk_end) {
      w.tile = (int)(sk_cur / p.kb_total);
      w.kb0 = (int)(sk_cur - (long long)w.tile * p.kb_total);
      w.kbn = (int)min((long long)(p.kb_total - w.kb0), sk_end - sk_cur);
      w.kstep = 1;
      sk_cur += w.kbn;
      raster_tile(p, w.tile, w.tp, w.tq);
      w.partial = w.kbn != p.kb_total;
      if (w.partial) {
        const int first = owner((long long)w.tile * p.kb_total);
        const int last = owner((long long)(w.tile + 1) * p.kb_total - 1);
        w.n_contrib = last - first + 1;
        w.slot0 = w.tile * p.sk_slots;
        w.slot = w.slot0 + (me - first);
      }
      return true;
    }
    if (p.sk_tiles > 0) {
      if (next_u >= p.num_tiles) return false;
      w.tile = next_u;
      next_u += count;
      raster_tile(p, w.tile, w.tp, w.tq);
      w.kb0 = 0, w.kbn = p.kb_total, w.kstep = 1, w.partial = 0;
      return true;
    }
    if (next_u >= p.num_units) return false;
    const int u = next_u;
    next_u += count;
    w.tile = u / p.split_k;
    const int slice = u - w.tile * p.split_k;
    raster_tile(p, w.tile, w.tp, w.tq);
    // Slice s takes K blocks s, s + split_k, ...: the slices of a tile run at the same time on neighbouring CTAs, so
    // together they walk every operand row front to back instead of starting at split_k distant offsets.
    w.kb0 = slice;
    w.kstep = p.split_k;
    w.kbn = (p.kb_total - slice + p.split_k - 1) / p.split_k;
    w.partial = p.split_k > 1;
    w.n_contrib = p.split_k;
    w.slot0 = w.tile * p.split_k;
    w.slot = w.slot0 + slice;
    return true;
  }
};

// CG = CTAs that share one output tile: 1, or 2 for a tcgen05 cta_group::2 pair (each CTA then holds 128 of the
// tile's 256 U rows and half of its V rows).
// TK = K elements per pipeline stage: 64, or 128 (two boxes per operand) for narrow tiles, where the fixed cost of a
// stage (barrier poll, election, commit) would otherwise exceed the few tensor cycles a 64-deep block needs.
template <int TILE_Q, int STAGES, int CG, int TK>
struct SmemLayout {
  static constexpr int kSub = TK / kBoxK;  // 64-deep boxes per operand and stage
  static constexpr int kVRows = TILE_Q / CG;
  // One tcgen05.mma covers at most 256 columns: a 512-wide tile takes two per K step, each reading kMmaVRows of this
  // CTA's V rows (half h of the tile = columns 256h .. 256h+255 of the accumulator).
  static constexpr int kHalves = TILE_Q > 256 ? 2 : 1;
  static constexpr int kMmaVRows = kVRows / kHalves;
  // An operand that is contiguous along its rows arrives in boxes of 64 rows: a CTA's share of 96 rows (the 192-wide
  // pair tile) then occupies two boxes, so the V part of a stage is sized for whole boxes.
  static constexpr int kVBoxRows = kVRows > 64 ? (kVRows + 63) / 64 * 64 : kVRows;
  static constexpr int kVBoxBytes = kVBoxRows * kBoxK * 2;
  static constexpr int kUStageBytes = kSub * kUBoxBytes;
  static constexpr int kVStageBytes = kSub * kVBoxBytes;
  static constexpr int kStageBytes = kUStageBytes + kVStageBytes;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  // Epilogue staging for TMA stores: per epilogue warp two 32-row x 128-byte swizzled images (tiles >= 64 wide only).
  static constexpr int kStageOutBytes = 32 * 128;
  static constexpr int kOutOff = kRingBytes;
  // In cluster split-K mode the other CTAs' rows arrive in float[S][128/S][TILE_Q]: in this region for tiles up to 64
  // wide; wider tiles reuse the operand ring instead (it is idle once the last MMA has completed).
  static constexpr bool kRecvInRing = TILE_Q > 64;
  static constexpr int kRecvOff = kRecvInRing ? 0 : kRingBytes;
  static constexpr int kRecvBytes = TILE_Q <= 64 ? kTileP * TILE_Q * 4 : 0;
  static constexpr int kStagingBytes = TILE_Q >= 64 ? 4 * 2 * kStageOutBytes : 0;
  static constexpr int kOutBytes = kRecvBytes > kStagingBytes ? kRecvBytes : kStagingBytes;
  static constexpr int kBiasOff = kOutOff + kOutBytes;   // float[256]; a 512-wide tile keeps its slice in 16 bits
  static constexpr int kBiasBytes = TILE_Q > 256 ? TILE_Q * 2 : 256 * 4;
  static constexpr int kBarOff = kBiasOff + kBiasBytes;  // full[S], empty[S], acc_full[2], acc_empty[2]
  static constexpr int kMiscOff = kBarOff + (2 * STAGES + 4) * 8;  // tmem ptr, abort flag, last flag, epilogue verdict
  static constexpr int kTotal = kMiscOff + 32;
  static constexpr int kDynBytes = kTotal + 1024;  // slack for manual 1024-byte alignment
};

constexpr int kTraceRoles = 4, kTraceItems = 16, kTraceStamps = 4;
__device__ __forceinline__ void trace_stamp(const GemmParams& p, int role, int item, int k) {
  if (p.trace != nullptr && item < kTraceItems)
    p.trace[(((size_t)blockIdx.x * kTraceRoles + role) * kTraceItems + item) * kTraceStamps + k] = globaltimer_ns();
}

__device__ __forceinline__ void trace_value(const GemmParams& p, int role, int item, int k, long long v) {
  if (p.trace != nullptr && item < kTraceItems)
    p.trace[(((size_t)blockIdx.x * kTraceRoles + role) * kTraceItems + item) * kTraceStamps + k] = (unsigned long long)v;
}

__device__ __forceinline__ void report_abort(const GemmParams& p, int role, int unit) {
  if (p.status != nullptr) {
    if (atomicCAS(p.status, 0, 1) == 0) {
      p.status[1] = blockIdx.x;
      p.status[2] = role;
      p.status[3] = unit;
    }
  }
}

// Add bias, cast and store one chunk of CW consecutive Q-columns of one P-row (BIAS_Q_DONE: the caller has already
// added the per-column bias).
template <int CW, bool BIAS_Q_DONE = false>
__device__ __forceinline__ void finalize_chunk(const GemmParams& p, float (&v)[CW], int prow, int q0,
                                               const float* bias_q /* smem, chunk-local */, float bias_p) {
  if (prow >= p.P) return;
  if (!p.swap_out) {
    if (!BIAS_Q_DONE && p.bias != nullptr) {
#pragma unroll
      for (int i = 0; i < CW; ++i) v[i] += bias_q[i];
    }
    const long long base = (long long)prow * p.ldo + q0;
    if (p.out_dtype == 1) {
      float* o = reinterpret_cast<float*>(p.out) + base;
      if (q0 + CW <= p.Q && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < CW; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < CW; ++i)
          if (q0 + i < p.Q) o[i] = v[i];
      }
    } else {
      uint32_t pk[CW / 2];
      if (p.out_dtype == 2) {
#pragma unroll
        for (int i = 0; i < CW; i += 2) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[i], v[i + 1]);
          pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
        }
      } else {
#pragma unroll
        for (int i = 0; i < CW; i += 2) {
          __half2 h = __floats2half2_rn(v[i], v[i + 1]);
          pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + base;
      if (q0 + CW <= p.Q && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < CW / 2; i += 4)
          *reinterpret_cast<uint4*>(o + 2 * i) = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < CW; ++i)
          if (q0 + i < p.Q) o[i] = static_cast<uint16_t>((i & 1) ? (pk[i / 2] >> 16) : (pk[i / 2] & 0xffffu));
      }
    }
  } else {
    // D^T: consecutive lanes hold consecutive p -> each scalar store is warp-coalesced along p.
#pragma unroll
    for (int i = 0; i < CW; ++i) {
      const int q = q0 + i;
      if (q < p.Q) {
        const float x = v[i] + bias_p;
        const long long idx = (long long)q * p.ldo + prow;
        if (p.out_dtype == 1) {
          reinterpret_cast<float*>(p.out)[idx] = x;
        } else if (p.out_dtype == 2) {
          reinterpret_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(x);
        } else {
          reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn(x);
        }
      }
    }
  }
}

__device__ __forceinline__ float load_in_as_float(const void* ptr, long long i, int in_dtype) {
  if (in_dtype == 2) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ptr)[i]);
  return __half2float(reinterpret_cast<const __half*>(ptr)[i]);
}

template <int TILE_Q, int STAGES, int CG, int TK, bool LOADER = false>
__global__ void __launch_bounds__(LOADER ? kThreadsLoader : kThreads, 1) gemm_a16w16_sm100_kernel(const __grid_constant__ GemmParams p) {
  using L = SmemLayout<TILE_Q, STAGES, CG, TK>;
  constexpr int CW = TILE_Q >= 32 ? 32 : 16;  // columns per tcgen05.ld
  constexpr int NCHUNK = TILE_Q / CW;
  // The 512-column variant takes the width of its tiles at run time (a multiple of 32 above 256): the host picks the
  // width that fills whole waves. Its second MMA then covers tile_q - 256 columns, read from the first
  // (tile_q - 256) / 2 rows of each CTA's second V box; the boxes themselves are always loaded whole.
  const int tile_q = TILE_Q > 256 ? p.tile_q : TILE_Q;
  const int nchunk = TILE_Q > 256 ? tile_q / CW : NCHUNK;
  // TMEM is allocated in powers of two of at least 32 columns: two accumulators of TILE_Q columns each
  // (a 512-wide tile fills all 512 columns with one accumulator: its epilogue does not overlap the next main loop)
  constexpr int kAccBufs = 2 * TILE_Q <= 512 ? 2 : 1;
  constexpr uint32_t kTmemCols = 2 * TILE_Q <= 32 ? 32 : 2 * TILE_Q <= 64 ? 64 : 2 * TILE_Q <= 128 ? 128 : 2 * TILE_Q <= 256 ? 256 : 512;
  // a pair's two CTAs both report to the leader's barrier; with loader warps only the TMA-fetched operand counts
  // (a K-contiguous V of 96 rows per CTA fills only three quarters of its two-box slot)
  const uint32_t tx_bytes = LOADER                      ? p.tma_tx_bytes
                            : L::kVBoxRows != L::kVRows ? (uint32_t)(CG * (L::kUStageBytes + L::kSub * (p.v_mn_major ? L::kVBoxBytes : L::kVRows * kBoxK * 2)))
                                                        : (uint32_t)(CG * L::kStageBytes);
  // arrivals that complete a stage: the producer's expect_tx, plus one per CTA from its loader warps
  constexpr uint32_t kFullArrivals = LOADER ? 1 + CG : 1;
  constexpr int kVRows = L::kVRows;
  constexpr int kMmaVRows = L::kMmaVRows;
  constexpr int kSlotVec = NCHUNK * (CW / 4) * kTileP;  // float4 per partial slot of one CTA

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);

  float* bias_s = reinterpret_cast<float*>(sm + L::kBiasOff);
  const uint32_t bar0 = base + L::kBarOff;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_ptr_s = reinterpret_cast<volatile uint32_t*>(sm + L::kMiscOff);
  volatile int* abort_s = reinterpret_cast<volatile int*>(sm + L::kMiscOff + 4);
  volatile int* last_s = reinterpret_cast<volatile int*>(sm + L::kMiscOff + 8);
  volatile int* epi_abort_s = reinterpret_cast<volatile int*>(sm + L::kMiscOff + 12);
  const unsigned long long wait_limit = p.wait_limit_ns;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = CG == 2 ? (int)cluster_ctarank() : 0;  // 0 = leader of the pair (issues the MMAs)
  const int walker = CG == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int walkers = CG == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), kFullArrivals);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accf_bar(b), 1);
      mbar_init(acce_bar(b), 4 * CG);  // one arrival per epilogue warp of every CTA of the pair
    }
    *abort_s = 0;
    *last_s = 0;
    *epi_abort_s = 0;
    *(epi_abort_s + 1) = 0;  // the loader warps' verdict word
    fence_mbar_init();
    if (!(LOADER && p.u_cp)) prefetch_tmap(&p.tmap_u);
    if (!(LOADER && p.v_cp)) prefetch_tmap(&p.tmap_v);
    if (p.tma_store) prefetch_tmap(&p.tmap_out);
  }
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(const_cast<uint32_t*>(tmem_ptr_s)), kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  __syncthreads();
  const bool cluster_mode = CG == 1 && p.cluster_split > 1;
  // Every CTA of a cluster must be running before anything is sent across it. A pair needs that before its first
  // load (the peer's barriers are signalled from the start); cluster split-K only before the epilogue's scatter, so
  // there each thread arrives now and waits later (`cluster_wait_due`), keeping the barrier off the load path.
  bool cluster_wait_due = false;
  // Wide tiles receive into the operand ring, so every CTA of the cluster must have finished its MMAs before anyone
  // scatters: one more cluster barrier ("ring idle"), owed by every thread exactly once.
  bool ring_idle_barrier_due = cluster_mode && L::kRecvInRing;
  if (CG == 2) {
    cluster_arrive();
    cluster_wait();
  } else if (cluster_mode) {
    cluster_arrive();
    cluster_wait_due = true;
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;
  // Everything above touched only this CTA's own shared memory, TMEM and kernel parameters, so with a programmatic
  // dependent launch it overlaps the tail of the previous kernel in the stream. From here on global memory is read
  // and written (operands may be that kernel's output; the workspace is shared with it).
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one per CTA)
    // Like the MMA warp, the whole warp walks the loop (uniform operands); lane 0 polls, one elected lane issues.
    {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      WorkIter wi;
      wi.init(p, walker, walkers);
      Unit w;
      int item = 0;
      // Requests of one K block: the U boxes and the V boxes of stage `st`, counted on barrier `fb`.
      auto load = [&](uint32_t dst, const void* map, int x, int y, uint32_t fb) {
        if constexpr (CG == 2)
          tma_load_2d_pair(dst, map, x, y, fb);
        else
          tma_load_2d(dst, map, x, y, fb);
      };
      auto load_u = [&](int st, int kb, int p0, uint32_t fb) {
        const uint32_t su = base + st * L::kStageBytes;
#pragma unroll
        for (int sub = 0; sub < L::kSub; ++sub) {
          const int k0 = kb * TK + sub * kBoxK;
          const uint32_t bu = su + sub * kUBoxBytes;
          if (!p.u_mn_major) {
            load(bu, &p.tmap_u, k0, p0, fb);
          } else {
            load(bu, &p.tmap_u, p0, k0, fb);
            load(bu + 8192u, &p.tmap_u, p0 + 64, k0, fb);
          }
        }
      };
      auto load_v = [&](int st, int kb, int q0, uint32_t fb) {
        const uint32_t sv = base + st * L::kStageBytes + L::kUStageBytes;
#pragma unroll
        for (int sub = 0; sub < L::kSub; ++sub) {
          const int k0 = kb * TK + sub * kBoxK;
          const uint32_t bv = sv + sub * L::kVBoxBytes;
          // first V row of accumulator half h: q0 for half 0; half 1 starts 256 columns into the tile and gives each
          // CTA (tile_q - 256) / 2 of its columns
          auto half_q0 = [&](int h) { return h == 0 ? q0 : q0 - rank * kMmaVRows + 256 + rank * ((tile_q - 256) >> 1); };
          if (!p.v_mn_major) {
#pragma unroll
            for (int h = 0; h < L::kHalves; ++h) load(bv + (uint32_t)(h * kMmaVRows * 128), &p.tmap_v, k0, half_q0(h), fb);
          } else {
            constexpr int kPerHalf = kMmaVRows >= 64 ? (kMmaVRows + 63) / 64 : 1;  // 64-row boxes per accumulator half
#pragma unroll
            for (int j = 0; j < (kVRows >= 64 ? (kVRows + 63) / 64 : 1); ++j)
              load(bv + 8192u * j, &p.tmap_v, half_q0(j / kPerHalf) + 64 * (j % kPerHalf), k0, fb);
          }
        }
      };
      // Data of both CTAs of a pair is counted on the leader's barrier, which the MMA thread waits on.
      auto full_target = [&](int st) {
        uint32_t fb = full_bar(st);
        if constexpr (CG == 2) fb = mapa_cluster(fb, 0);
        return fb;
      };
      // In the first pass over the ring every stage is free: no need to ask its barrier.
#pragma unroll 1
      for (; ok && wi.next(p, w); ++item) {
        const int u = w.tile;
        // the pair's MMA reads rows 0..kMmaVRows-1 of each CTA's V stage as columns rank * kMmaVRows .. of the accumulator
        const int p0 = (w.tp * CG + rank) * kTileP, q0 = w.tq * tile_q + rank * kMmaVRows;
        if (lane == 0) {
          trace_stamp(p, 0, item, 0);
          trace_value(p, 0, item, 3, clock64());  // with the epilogue's pair of the same kind: the SM clock of this run
        }
#pragma unroll 1
        for (int kj = 0; kj < w.kbn; ++kj) {
          const int kb = w.kb0 + kj * w.kstep;
          if (issued >= STAGES) {
            int good = 1;
            if (lane == 0) good = mbar_wait<CG == 2>(empty_bar(stage), phase ^ 1u, abort_s, wait_limit) ? 1 : 0;
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) {
              if (lane == 0) report_abort(p, 0, u);
              ok = false;
              break;
            }
          }
          if (kj == 0 && lane == 0) trace_stamp(p, 0, item, 1);
          const uint32_t fb = full_target(stage);
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), tx_bytes);
            if (!(LOADER && p.u_cp)) load_u(stage, kb, p0, fb);
            if (!(LOADER && p.v_cp)) load_v(stage, kb, q0, fb);
          }
          __syncwarp();
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (lane == 0) trace_stamp(p, 0, item, 2);
      }
      if (!ok && lane == 0) {
        if (CG == 1) {
          // Loads already issued still write this CTA's smem: give each one a bounded chance to land.
          const int pending = issued < STAGES ? issued : STAGES;
          for (int i = 0; i < pending; ++i) {
            int s = stage - 1 - i;
            uint32_t ph = phase;
            if (s < 0) {
              s += STAGES;
              ph ^= 1u;
            }
            const unsigned long long t0 = globaltimer_ns();
            while (!mbar_try_wait(full_bar(s), ph) && globaltimer_ns() - t0 < 100000000ull) {
            }
          }
        } else {
          // In a pair the byte counts live on the leader's barriers: wait a fixed, bounded time instead.
          const unsigned long long t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 1000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (the pair's leader only)
    // The whole warp walks the loop so that control flow and operands stay warp-uniform; lane 0 polls the
    // barriers and the verdict is broadcast, one elected lane issues the tensor-core instructions.
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      WorkIter wi;
      wi.init(p, walker, walkers);
      Unit w;
      const bool tracing = p.trace != nullptr && p.trace_detail != 0;
      // `ready` = the full barrier of the stage about to be consumed was already seen complete (probed one K block
      // ahead, so that the probe's latency hides behind the MMA issue of the block before).
      int ready = 0;
#pragma unroll 1
      for (; ok && wi.next(p, w); ++it) {
        const int u = w.tile;
        const int buf = kAccBufs == 2 ? (it & 1) : 0;
        const uint32_t acc_phase = (kAccBufs == 2 ? (it >> 1) : it) & 1;
        int good = 1;
        if (lane == 0) good = mbar_wait<CG == 2>(acce_bar(buf), acc_phase ^ 1u, abort_s, wait_limit) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          if (lane == 0) report_abort(p, 1, u);
          break;
        }
        tc_fence_after();
        if (lane == 0) trace_stamp(p, 1, it, 0);
        int stalls = 0;
        long long c_wait = 0, c_mma = 0, c_commit = 0;
        const uint32_t d_tmem = tmem_base + buf * TILE_Q;
#pragma unroll 1
        for (int kb = 0; kb < w.kbn; ++kb) {
          long long c0 = 0, c1 = 0, c3 = 0;
          if (tracing) c0 = clock64();
          if (!ready) {
            if (lane == 0) {
              ++stalls;
              good = mbar_wait<CG == 2>(full_bar(stage), phase, abort_s, wait_limit) ? 1 : 0;
            }
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) {
              if (lane == 0) report_abort(p, 2, u);
              ok = false;
              break;
            }
          }
          tc_fence_after();
          if (tracing) c1 = clock64();
          if (kb == 0 && lane == 0) trace_stamp(p, 1, it, 1);
          const uint32_t su = base + stage * L::kStageBytes;
          const uint32_t sv = su + L::kUStageBytes;
          // Probe the next stage now; the answer is collected after the MMAs below have been issued.
          const int nstage = stage + 1 == STAGES ? 0 : stage + 1;
          const uint32_t nphase = stage + 1 == STAGES ? phase ^ 1u : phase;
          int next_ready = 0;
          if (lane == 0) next_ready = mbar_try_wait(full_bar(nstage), nphase) ? 1 : 0;
          if (elect_one()) {
#pragma unroll
            for (int sub = 0; sub < L::kSub; ++sub) {
              const uint32_t bu = su + sub * kUBoxBytes, bv = sv + sub * L::kVBoxBytes;
              const uint64_t du = (uint64_t(p.u_desc_hi) << 32) | uint64_t(p.u_desc_lo | ((bu >> 4) & 0x3fffu));
              const uint64_t dv = (uint64_t(p.v_desc_hi) << 32) | uint64_t(p.v_desc_lo | ((bv >> 4) & 0x3fffu));
#pragma unroll
              for (int j = 0; j < kBoxK / kUmmaK; ++j) {
#pragma unroll
                for (int h = 0; h < L::kHalves; ++h)
                  umma_f16<CG>(d_tmem + (uint32_t)(h * 256), du + uint64_t(j * p.u_kstep),
                               dv + uint64_t(j * p.v_kstep + h * ((kMmaVRows * 128) >> 4)), h == 0 ? p.idesc : p.idesc2,
                               (kb | sub | j) != 0 ? 1u : 0u);
              }
            }
            if (tracing) c3 = clock64();
            // Frees the stage, in every CTA of the pair, once these MMAs have read it.
            if constexpr (CG == 2) {
              umma_commit_pair(mapa_cluster(empty_bar(stage), 0));
              umma_commit_pair(mapa_cluster(empty_bar(stage), 1));
            } else {
              umma_commit(empty_bar(stage));
            }
            if (tracing) {
              const long long c4 = clock64();
              c_wait += c1 - c0, c_mma += c3 - c1, c_commit += c4 - c3;
            }
          }
          ready = __shfl_sync(0xffffffffu, next_ready, 0);
          stage = nstage;
          phase = nphase;
        }
        if (elect_one()) {
          trace_stamp(p, 1, it, 2);
          trace_value(p, 1, it, 3, stalls);
          if (tracing) {
            trace_value(p, 3, it, 0, c_wait);
            trace_value(p, 3, it, 2, c_mma);
            trace_value(p, 3, it, 3, c_commit);
          }
          if (ok) {  // accumulator complete: wake the epilogue of every CTA of the pair
            if constexpr (CG == 2) {
              umma_commit_pair(mapa_cluster(accf_bar(buf), 0));
              umma_commit_pair(mapa_cluster(accf_bar(buf), 1));
            } else {
              umma_commit(accf_bar(buf));
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (!LOADER || warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of every CTA)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;
    const int et = threadIdx.x - 64;  // 0..127
    int it = 0;
    int out_flip = 0;  // which of the warp's two staging images the next TMA store uses
    WorkIter wi;
    wi.init(p, walker, walkers);
    Unit w;
#pragma unroll 1
    for (; wi.next(p, w); ++it) {
      const int u = w.tile;
      const int buf = kAccBufs == 2 ? (it & 1) : 0;
      const uint32_t acc_phase = (kAccBufs == 2 ? (it >> 1) : it) & 1;
      const int prow = (w.tp * CG + rank) * kTileP + row;
      const int qbase = w.tq * tile_q;
      const bool direct = !w.partial;

      // Stage the bias slice of this tile (columns of D) while the main loop runs.
      float bias_p = 0.f;
      if (p.bias != nullptr) {
        if (!p.swap_out) {
          named_bar_sync(1, kEpiThreads);  // previous unit finished reading bias_s
          for (int i = et; i < tile_q; i += kEpiThreads) {
            const int q = qbase + i;
            if constexpr (TILE_Q > 256)  // kept as the 16 input bits (zero bits are 0.0 in both formats)
              reinterpret_cast<uint16_t*>(bias_s)[i] = q < p.Q ? reinterpret_cast<const uint16_t*>(p.bias)[q] : (uint16_t)0;
            else
              bias_s[i] = q < p.Q ? load_in_as_float(p.bias, q, p.in_dtype) : 0.f;
          }
          named_bar_sync(1, kEpiThreads);
        } else if (prow < p.P) {
          bias_p = load_in_as_float(p.bias, prow, p.in_dtype);
        }
      }

      // Every thread polls for itself (only the time limit ends its wait). A thread whose limit ran out says so in
      // shared memory before it leaves; one that saw the barrier complete later finds that note and leaves too, so
      // that either all 128 threads go on to the named barriers below or none does.
      if (!mbar_wait<CG == 2, false>(accf_bar(buf), acc_phase, abort_s, wait_limit)) {
        *epi_abort_s = 1;
        report_abort(p, 3, u);
        break;
      }
      if (*epi_abort_s != 0) break;
      tc_fence_after();
      if (et == 0) {
        trace_stamp(p, 2, it, 0);
        trace_value(p, 2, it, 3, clock64());
      }
      const uint32_t t_acc = tmem_base + buf * TILE_Q + (uint32_t(quarter * 32) << 16);
      float4* part = nullptr;
      if (!direct) part = reinterpret_cast<float4*>(p.partials) + (size_t)(w.slot * CG + rank) * kSlotVec + row;
      // Two register buffers: the tcgen05.ld of chunk c+1 is in flight while chunk c is converted and stored.
      auto load_chunk = [&](uint32_t(&r)[32], int c) {
        if constexpr (CW == 32)
          tmem_ld_32x32(t_acc + c * CW, r);
        else
          tmem_ld_32x16(t_acc + c * CW, r);
      };
      auto release_acc = [&]() {
        // Everything this warp needs is in registers: hand the accumulator back to the MMA thread.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CG == 2 && rank != 0)
            mbar_arrive_cluster(acce_bar(buf), 0);
          else
            mbar_arrive(acce_bar(buf));
        }
      };
      uint32_t cl_stage = 0;
      if (cluster_mode) {
        if (cluster_wait_due) {
          cluster_wait();
          cluster_wait_due = false;
        }
        if (ring_idle_barrier_due) {  // this CTA's accumulator is complete, so its ring is idle: tell the cluster
          cluster_arrive();
          cluster_wait();
          ring_idle_barrier_due = false;
        }
        // Scatter staging: 32 rows x CW floats per epilogue warp. Wide tiles use the TMA-store staging area (unused in
        // this mode); narrower ones the head of this CTA's own ring, idle now that its accumulator is complete.
        cl_stage = base + (L::kRecvInRing ? L::kOutOff : 0) + (uint32_t)(warp - 2) * (32u * CW * 4u);
      }
      // TMA-store path: bias + cast, then this lane's row segment goes into the warp's swizzled staging image
      // (16-byte chunk j of row t sits at position j ^ (t % 8)); every full 128-byte row image is stored by one lane.
      // K-parallel units of the atomic mode leave like whole tiles, except that their boxes are added to C
      const bool red = !direct && p.atomic_out != 0;
      const bool staged = (direct || red) && p.tma_store != 0 && TILE_Q >= 64;
      // The warp normally alternates between two 4 KB staging images and waits for the TMA store that last read one
      // before rewriting it. In a CTA's last work item nothing will be loaded into the operand ring any more and the
      // accumulator being complete means the ring has been read: every flush then gets an image of its own in the ring
      // and never waits (the exposed epilogue at the end of the kernel is otherwise bound by TMA-store round trips).
      // at most one flush per chunk (fp32 output); a 512-wide tile of 16-bit output counts its real one per two chunks
      const int kFlushesPerTile = (TILE_Q > 256 && p.out_dtype != 1) ? (nchunk + 1) / 2 : nchunk;
      const bool tail_stage = L::kRingBytes >= 4 * kFlushesPerTile * L::kStageOutBytes && !wi.more(p);
      const uint32_t out_stage0 = tail_stage ? base + (uint32_t)(warp - 2) * (uint32_t)(kFlushesPerTile * L::kStageOutBytes)
                                             : base + L::kOutOff + (uint32_t)(warp - 2) * (2 * L::kStageOutBytes);
      if (tail_stage) out_flip = 0;
      auto stage_image = [&]() -> uint32_t {
        return out_stage0 + (uint32_t)(tail_stage ? out_flip : (out_flip & 1)) * L::kStageOutBytes;
      };
      auto stage_flush = [&](int col0) {
        fence_proxy_async_smem();
        __syncwarp();
        const int row0 = (w.tp * CG + rank) * kTileP + quarter * 32;
        if (lane == 0) {
          // a box that starts outside C holds nothing to write; one that straddles the edge is clipped by TMA
          if (row0 < p.P && col0 < p.Q) {
            if (red)
              tma_reduce_add_2d(&p.tmap_out, col0, row0, stage_image());
            else
              tma_store_2d(&p.tmap_out, col0, row0, stage_image());
          }
          tma_store_commit();
        }
        ++out_flip;
      };
      auto stage_acquire = [&]() {
        // the store issued two flushes ago has finished reading the buffer about to be overwritten
        if (tail_stage) return;  // every flush of a CTA's last work item has its own image
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
      };
      // Adds the bias of the CW columns of chunk c, from the 16-bit slice a 512-wide tile keeps.
      auto add_bias16 = [&](int c, auto& v, int off) {  // v[off .. off + CW) are the chunk's values
        const uint4* s16 = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(bias_s) + c * CW);
#pragma unroll
        for (int j = 0; j < CW / 8; ++j) {
          const uint4 x = s16[j];
          const uint32_t wds[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            if (p.in_dtype == 2) {
              v[off + 8 * j + 2 * t] += __uint_as_float(wds[t] << 16);
              v[off + 8 * j + 2 * t + 1] += __uint_as_float(wds[t] & 0xffff0000u);
            } else {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wds[t]));
              v[off + 8 * j + 2 * t] += f.x, v[off + 8 * j + 2 * t + 1] += f.y;
            }
          }
        }
      };
      auto finalize = [&](float(&v)[CW], int c) {
        if constexpr (TILE_Q > 256) {
          if (p.bias != nullptr && !p.swap_out) add_bias16(c, v, 0);
          finalize_chunk<CW, true>(p, v, prow, qbase + c * CW, nullptr, bias_p);
        } else {
          finalize_chunk<CW>(p, v, prow, qbase + c * CW, bias_s + c * CW, bias_p);
        }
      };
      auto process_chunk = [&](uint32_t(&r)[32], int c) {
        float v[CW];
#pragma unroll
        for (int i = 0; i < CW; ++i) v[i] = __uint_as_float(r[i]);
        if (TILE_Q < 128 && staged) {  // (tiles of 128 columns and more take the 64-column steps below)
          if constexpr (CW == 32) {
            if constexpr (TILE_Q > 256) {
              if (p.bias != nullptr && !red) add_bias16(c, v, 0);
            } else if (p.bias != nullptr && !red) {  // in the atomic mode C already holds the bias
              const float4* b4 = reinterpret_cast<const float4*>(bias_s + c * CW);  // 16-byte aligned: one load per 4 columns
#pragma unroll
              for (int j = 0; j < CW / 4; ++j) {
                const float4 b = b4[j];
                v[4 * j] += b.x, v[4 * j + 1] += b.y, v[4 * j + 2] += b.z, v[4 * j + 3] += b.w;
              }
            }
            const uint32_t row_base = stage_image() + (uint32_t)lane * 128u;
            if (p.out_dtype == 1) {
              stage_acquire();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t addr = row_base + (uint32_t)((j ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]),
                             "f"(v[4 * j + 3])
                             : "memory");
              }
              stage_flush(qbase + c * CW);
            } else {
              if ((c & 1) == 0) stage_acquire();
              uint32_t pk[16];
              if (p.out_dtype == 2) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[i], v[i + 1]);
                  pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  __half2 h = __floats2half2_rn(v[i], v[i + 1]);
                  pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int jj = (c & 1) * 4 + j;
                const uint32_t addr = row_base + (uint32_t)((jj ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * j]), "r"(pk[4 * j + 1]), "r"(pk[4 * j + 2]),
                             "r"(pk[4 * j + 3])
                             : "memory");
              }
              if (c & 1) stage_flush(qbase + (c - 1) * CW);
            }
          }
        } else if (direct) {
          finalize(v, c);
        } else if (cluster_mode) {
          // cluster split-K: the partial sums of row r go to the CTA that owns r, into its image
          // recv[source rank][chunk][r % R][CW]. A lane holds one row, so the warp first transposes through its staging
          // image (16-byte piece j of row t at position j ^ (t % 8), conflict-free) and then copies it out with every
          // warp-wide store covering whole 128-byte rows: remote shared-memory stores are only fast when coalesced.
          constexpr int kPieces = CW / 4;             // 16-byte pieces per row of a chunk
          constexpr int kRowsPerStep = 32 / kPieces;  // rows one warp-wide store covers
          const uint32_t my_row = cl_stage + (uint32_t)lane * (CW * 4u);
#pragma unroll
          for (int j = 0; j < kPieces; ++j) {
            const uint32_t addr = my_row + (uint32_t)((j ^ (lane & (kPieces - 1))) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]),
                         "f"(v[4 * j + 3])
                         : "memory");
          }
          __syncwarp();
          const int R = kTileP / p.cluster_split;
          const uint32_t recv_chunk = base + L::kRecvOff + (uint32_t)(((int)cluster_ctarank() * NCHUNK + c) * R) * (CW * 4u);
#pragma unroll
          for (int step = 0; step < kPieces; ++step) {
            const int t = step * kRowsPerStep + lane / kPieces;  // row inside this warp's 32
            const uint32_t piece = (uint32_t)(lane % kPieces) << 4;
            float4 x;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                         : "r"(cl_stage + (uint32_t)t * (CW * 4u) + piece)
                         : "memory");
            const int trow = quarter * 32 + t;
            const uint32_t dst = mapa_cluster(recv_chunk + (uint32_t)(trow % R) * (CW * 4u) + piece, (uint32_t)(trow / R));
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w)
                         : "memory");
          }
          __syncwarp();  // the staging image is rewritten by the next chunk
        } else {
          // slot layout [chunk][4-column group][row][4]: one warp store covers 512 contiguous bytes
          float4* dst = part + (size_t)c * (CW / 4) * kTileP;
#pragma unroll
          for (int j = 0; j < CW / 4; ++j)
            __stcg(dst + j * kTileP, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
        }
      };
      bool done = false;
      // Two register buffers for tcgen05.ld, declared once for all the loops below: with buffers of their own per
      // loop the compiler spilled values that the producer's and the MMA issuer's loops use (config 5: +20 %).
      uint32_t ra[32], rb[32];
      if constexpr (CW == 32 && TILE_Q >= 128) {
        // The common exit (whole tile, 16-bit output, TMA stores) takes 64 columns per step in one straight-line
        // block: two tcgen05.ld, one wait, bias, cast, the lane's 128-byte row segment into the warp's swizzled
        // staging image, one flush. The loads of the next step are issued once this step's values have left the
        // registers and fly during the flush. (The 512-column variant needs it most: its single accumulator leaves
        // every epilogue unhidden.)
        if (staged && !red && p.out_dtype != 1) {
          done = true;
          const int nstep = nchunk >> 1;
          const bool lone = (nchunk & 1) != 0;  // a run-time width may leave one last chunk without a partner
          load_chunk(ra, 0);
          load_chunk(rb, 1);
#pragma unroll 1
          for (int sp = 0; sp < nstep; ++sp) {
            tmem_ld_wait();
            const bool more = sp + 1 < nstep;
            if (!more && !lone) release_acc();
            uint32_t pk[32];
            auto half = [&](uint32_t(&r)[32], int h) {  // 32 columns: bias, cast, pack into pk[16h .. 16h + 16)
              float v[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
              if (p.bias != nullptr) {
                if constexpr (TILE_Q > 256) {
                  add_bias16(2 * sp + h, v, 0);
                } else {
                  const float4* b4 = reinterpret_cast<const float4*>(bias_s + sp * 64 + h * 32);  // 16-byte aligned
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const float4 b = b4[j];
                    v[4 * j] += b.x, v[4 * j + 1] += b.y, v[4 * j + 2] += b.z, v[4 * j + 3] += b.w;
                  }
                }
              }
              if (p.out_dtype == 2) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  __nv_bfloat162 x = __floats2bfloat162_rn(v[i], v[i + 1]);
                  pk[16 * h + i / 2] = *reinterpret_cast<uint32_t*>(&x);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  __half2 x = __floats2half2_rn(v[i], v[i + 1]);
                  pk[16 * h + i / 2] = *reinterpret_cast<uint32_t*>(&x);
                }
              }
            };
            half(ra, 0);
            half(rb, 1);
            stage_acquire();
            const uint32_t row_base = stage_image() + (uint32_t)lane * 128u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t addr = row_base + (uint32_t)((j ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * j]), "r"(pk[4 * j + 1]), "r"(pk[4 * j + 2]),
                           "r"(pk[4 * j + 3])
                           : "memory");
            }
            if (more) {
              load_chunk(ra, 2 * sp + 2);
              load_chunk(rb, 2 * sp + 3);
            } else if (lone) {
              load_chunk(ra, nchunk - 1);
            }
            stage_flush(qbase + sp * 64);
          }
          if (lone) {  // no partner to fill a 128-byte row with: direct stores
            tmem_ld_wait();
            release_acc();
            float v[CW];
#pragma unroll
            for (int i = 0; i < CW; ++i) v[i] = __uint_as_float(ra[i]);
            finalize(v, nchunk - 1);
          }
        } else if (staged) {
          // fp32 rows (whole tiles, and the partial tiles of the atomic mode): the same steps, one 32-column image
          // and one flush per half
          done = true;
          const int nstep = nchunk >> 1;
          const bool lone = (nchunk & 1) != 0;
          auto half32 = [&](uint32_t(&r)[32], int c) {  // chunk c: bias, the lane's 128-byte row segment, flush
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            if (p.bias != nullptr && !red) {  // in the atomic mode C already holds the bias
              if constexpr (TILE_Q > 256) {
                add_bias16(c, v, 0);
              } else {
                const float4* b4 = reinterpret_cast<const float4*>(bias_s + c * CW);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 b = b4[j];
                  v[4 * j] += b.x, v[4 * j + 1] += b.y, v[4 * j + 2] += b.z, v[4 * j + 3] += b.w;
                }
              }
            }
            stage_acquire();
            const uint32_t row_base = stage_image() + (uint32_t)lane * 128u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t addr = row_base + (uint32_t)((j ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]),
                           "f"(v[4 * j + 3])
                           : "memory");
            }
          };
          load_chunk(ra, 0);
          load_chunk(rb, 1);
#pragma unroll 1
          for (int sp = 0; sp < nstep; ++sp) {
            tmem_ld_wait();
            const bool more = sp + 1 < nstep;
            if (!more && !lone) release_acc();
            half32(ra, 2 * sp);
            stage_flush(qbase + sp * 64);
            half32(rb, 2 * sp + 1);
            if (more) {
              load_chunk(ra, 2 * sp + 2);
              load_chunk(rb, 2 * sp + 3);
            } else if (lone) {
              load_chunk(ra, nchunk - 1);
            }
            stage_flush(qbase + sp * 64 + 32);
          }
          if (lone) {
            tmem_ld_wait();
            release_acc();
            half32(ra, nchunk - 1);
            stage_flush(qbase + (nchunk - 1) * CW);
          }
        }
      }
      if (!done) {
        load_chunk(ra, 0);
        tmem_ld_wait();
#pragma unroll 1
        for (int c = 0; c < nchunk; c += 2) {
          if (c + 1 < nchunk)
            load_chunk(rb, c + 1);
          else
            release_acc();
          process_chunk(ra, c);
          if (c + 1 < nchunk) {
            tmem_ld_wait();
            if (c + 2 < nchunk)
              load_chunk(ra, c + 2);
            else
              release_acc();
            process_chunk(rb, c + 1);
            if (c + 2 < nchunk) tmem_ld_wait();
          }
        }
      }

      if (et == 0) trace_stamp(p, 2, it, 1);
      if (!direct && !cluster_mode && !red) {
        // Ticket: the CTA that arrives last at this (half-)tile sums all contributions in slot order.
        // One thread fences for the group: the barrier orders every epilogue thread's partial stores before its
        // fence (release, cumulative), and its second fence (acquire) plus the barrier orders the reads after.
        named_bar_sync(2, kEpiThreads);
        if (et == 0) {
          int* ticket = p.tickets + (w.tile * CG + rank);
          __threadfence();
          const int t = atomicAdd(ticket, 1);
          __threadfence();
          const int last = (t == w.n_contrib - 1) ? 1 : 0;
          if (last) *ticket = 0;  // self-cleaning: nobody else touches it until the next launch
          *last_s = last;
        }
        named_bar_sync(2, kEpiThreads);
        const int last = *last_s;
        if (last) {
          const float4* tp0 = reinterpret_cast<const float4*>(p.partials) + (size_t)(w.slot0 * CG + rank) * kSlotVec + row;
          constexpr int kBatch = 4;  // contributors whose loads are in flight together
#pragma unroll 1
          for (int c = 0; c < nchunk; ++c) {
            float v[CW];
#pragma unroll
            for (int i = 0; i < CW; ++i) v[i] = 0.f;
#pragma unroll 1
            for (int s0 = 0; s0 < w.n_contrib; s0 += kBatch) {
              float4 x[kBatch][CW / 4];
#pragma unroll
              for (int bb = 0; bb < kBatch; ++bb) {
                if (s0 + bb < w.n_contrib) {
                  const float4* src = tp0 + (size_t)(s0 + bb) * (CG * kSlotVec) + (size_t)c * ((CW / 4) * kTileP);
#pragma unroll
                  for (int jj = 0; jj < CW / 4; ++jj) x[bb][jj] = __ldcg(src + jj * kTileP);
                }
              }
#pragma unroll
              for (int bb = 0; bb < kBatch; ++bb) {
                if (s0 + bb < w.n_contrib) {
#pragma unroll
                  for (int jj = 0; jj < CW / 4; ++jj) {
                    v[4 * jj] += x[bb][jj].x;
                    v[4 * jj + 1] += x[bb][jj].y;
                    v[4 * jj + 2] += x[bb][jj].z;
                    v[4 * jj + 3] += x[bb][jj].w;
                  }
                }
              }
            }
            finalize(v, c);
          }
        }
        named_bar_sync(2, kEpiThreads);  // last_s may be rewritten by the next unit
      }
      if (et == 0) trace_stamp(p, 2, it, 2);
    }
    if (lane == 0) tma_store_wait_all<0>();  // staging smem and C must be complete before the CTA leaves
  } else if constexpr (LOADER) {
    // ------------------------------------------------------------------ cp.async loaders (warps 6 and 7)
    // Thread t copies the 16-byte piece t%8 of rows t/8, t/8 + 8, ... of every box: eight neighbouring threads read
    // one 128-byte run of a row. Piece j of row r lands at position j ^ (r % 8) of the row's 128 bytes, which is
    // where a SWIZZLE_128B tensor-map copy puts it (boxes start on 1024-byte boundaries). Rows past the operand's
    // extent and K elements past K are zero-filled through the copy's source size, so nothing outside the logical
    // matrix is ever read. A source that is only 8-byte aligned (odd rows of a pitch that is 8 mod 16) takes two
    // 8-byte copies. The copies are plain (generic-proxy) writes: each thread waits for its own copies of a K
    // block, fences them towards the async proxy that tcgen05.mma reads through, the two warps meet at a named
    // barrier and one thread arrives on the stage's `full` barrier (the pair leader's, for both CTAs of a pair).
    // A block is signalled kLag blocks after it was issued, so that several blocks of copies are in flight.
    constexpr int kLag = STAGES - 1 < 3 ? STAGES - 1 : 3;
    const int lt = threadIdx.x - kThreads;
    const int lrow = lt >> 3, lj = lt & 7;
    const uint32_t dst_off = (uint32_t)lrow * 128u + (uint32_t)((lj ^ (lrow & 7)) << 4);
    volatile int* ld_abort_s = epi_abort_s + 1;  // shared word of the loader warps (zeroed with the other flags at kernel start)
    auto issue_box = [&](uint32_t box, const char* src0, long long pitch, int row0, int row_limit, int k0, int nrows) {
      const int kk = k0 + lj * 8;  // first K element of this thread's piece
      int kbytes = (p.K - kk) * 2;
      kbytes = kbytes < 0 ? 0 : (kbytes > 16 ? 16 : kbytes);
      for (int i = 0; i < nrows / 8; ++i) {
        const int r = row0 + lrow + 8 * i;
        const int nbytes = r < row_limit ? kbytes : 0;
        const char* src = nbytes > 0 ? src0 + (long long)r * pitch + (long long)kk * 2 : src0;
        const uint32_t dst = box + dst_off + (uint32_t)i * 1024u;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
          cp_async_16(dst, src, nbytes);
        } else {
          const int hi = nbytes - 8;
          cp_async_8(dst, src, nbytes < 8 ? nbytes : 8);
          cp_async_8(dst + 8u, hi > 0 ? src + 8 : src0, hi > 0 ? hi : 0);
        }
      }
    };
    int stage = 0, sig_stage = 0, pending = 0, issued = 0;
    uint32_t phase = 0;
    bool ok = true;
    WorkIter wi;
    wi.init(p, walker, walkers);
    Unit w;
    auto signal_oldest = [&]() {  // all loader threads call this together, after their own wait + fence
      named_bar_sync(4, kLoaderThreads);
      if (lt == 0) {
        if constexpr (CG == 2)
          mbar_arrive_cluster(full_bar(sig_stage), 0);
        else
          mbar_arrive(full_bar(sig_stage));
      }
      if (++sig_stage == STAGES) sig_stage = 0;
      --pending;
    };
#pragma unroll 1
    for (; ok && wi.next(p, w);) {
      const int p0 = (w.tp * CG + rank) * kTileP, q0 = w.tq * TILE_Q + rank * kVRows;
#pragma unroll 1
      for (int kj = 0; kj < w.kbn; ++kj) {
        const int kb = w.kb0 + kj * w.kstep;
        if (issued >= STAGES) {
          // One lane per warp polls (time limit only); the verdict is made common to the loader warps through shared
          // memory and a named barrier, so that they leave together or not at all.
          if (lane == 0 && !mbar_wait<CG == 2, false>(empty_bar(stage), phase ^ 1u, abort_s, wait_limit)) *ld_abort_s = 1;
          named_bar_sync(5, kLoaderThreads);
          if (*ld_abort_s != 0) {
            if (lt == 0) report_abort(p, 4, w.tile);
            ok = false;
            break;
          }
        }
        const uint32_t su = base + stage * L::kStageBytes;
        const uint32_t sv = su + L::kUStageBytes;
#pragma unroll
        for (int sub = 0; sub < L::kSub; ++sub) {
          const int k0 = kb * TK + sub * kBoxK;
          if (p.u_cp) issue_box(su + sub * kUBoxBytes, reinterpret_cast<const char*>(p.u_src), p.u_pitch, p0, p.P, k0, kTileP);
          if (p.v_cp) issue_box(sv + sub * L::kVBoxBytes, reinterpret_cast<const char*>(p.v_src), p.v_pitch, q0, p.Q, k0, kVRows);
        }
        cp_async_commit();
        ++pending;
        ++issued;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        if (pending > kLag) {
          cp_async_wait<kLag>();
          fence_proxy_async_smem();
          signal_oldest();
        }
      }
    }
    cp_async_wait<0>();  // every copy of this thread has landed (also when the loop was left early)
    if (ok) {
      fence_proxy_async_smem();
      while (pending > 0) signal_oldest();
    }
  }

  // ---------------------------------------------------------------------- teardown
  // Cluster barriers that this thread still owes come BEFORE the CTA-wide barrier: the epilogue warps pass them inside
  // their loop, so a producer / MMA warp that first waited for them at __syncthreads would never arrive (deadlock).
  if (cluster_wait_due) cluster_wait();  // warps that did not take part in the scatter still owe the first wait
  if (ring_idle_barrier_due) {           // ... and the "ring idle" barrier
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_before();
  __syncthreads();
  if (CG == 2 || cluster_mode) {
    // pair: no CTA leaves while its peer may still signal it or use its TMEM half;
    // cluster split-K: every CTA's rows have arrived in their owner's shared memory
    cluster_arrive();
    cluster_wait();
  }
  if constexpr (CG == 1) {
    if (cluster_mode && warp >= 2 && warp < 6) {  // the epilogue warps (a LOADER variant has two more warps behind them)
      // Each CTA owns R = 128/S rows of the tile: sum the S slabs in rank order (deterministic), bias, cast, store.
      const int S = p.cluster_split, R = kTileP / S;
      const int crank = (int)cluster_ctarank();
      const int tile = (int)blockIdx.x / S;
      int tp, tq;
      raster_tile(p, tile, tp, tq);
      const float* recv = reinterpret_cast<const float*>(sm + L::kRecvOff);
      const int et = threadIdx.x - 64;
      auto emit = [&](float acc, int prow, int q) {
        if (prow < p.P && q < p.Q) {
          if (p.bias != nullptr) acc += load_in_as_float(p.bias, p.swap_out ? prow : q, p.in_dtype);
          const long long idx = p.swap_out ? (long long)q * p.ldo + prow : (long long)prow * p.ldo + q;
          if (p.out_dtype == 1)
            reinterpret_cast<float*>(p.out)[idx] = acc;
          else if (p.out_dtype == 2)
            reinterpret_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(acc);
          else
            reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn(acc);
        }
      };
      constexpr int kPieces = CW / 4;  // 16-byte pieces per row of a chunk; piece j of row t sits at j ^ (t % kPieces)
      if (!p.swap_out) {
        // four consecutive columns per thread and step: float4 reads of the slabs, bias from the staged slice,
        // one 8- or 16-byte store (scalar stores at ragged edges or unaligned rows)
        const int es = p.out_dtype == 1 ? 4 : 2;
#pragma unroll 2
        for (int e = et; e < R * (TILE_Q / 4); e += kEpiThreads) {
          const int lrow = e / (TILE_Q / 4), g = e % (TILE_Q / 4), col = g * 4;
          const int off = ((g / kPieces) * R + lrow) * CW + (((g % kPieces) ^ (lrow & (kPieces - 1))) << 2);
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int src = 0; src < S; ++src) {
            const float4 x = *reinterpret_cast<const float4*>(recv + src * (R * TILE_Q) + off);
            acc.x += x.x, acc.y += x.y, acc.z += x.z, acc.w += x.w;
          }
          const int prow = tp * kTileP + crank * R + lrow, q = tq * TILE_Q + col;
          if (prow >= p.P || q >= p.Q) continue;
          if (p.bias != nullptr) acc.x += bias_s[col], acc.y += bias_s[col + 1], acc.z += bias_s[col + 2], acc.w += bias_s[col + 3];
          char* dst = reinterpret_cast<char*>(p.out) + ((long long)prow * p.ldo + q) * es;
          if (q + 3 < p.Q && (reinterpret_cast<uintptr_t>(dst) & (uintptr_t)(4 * es - 1)) == 0) {
            if (p.out_dtype == 1) {
              *reinterpret_cast<float4*>(dst) = acc;
            } else if (p.out_dtype == 2) {
              __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
              *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
              __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
              *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
          } else {
            const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int t = 0; t < 4; ++t) {
              if (q + t < p.Q) {
                const long long idx = (long long)prow * p.ldo + q + t;
                if (p.out_dtype == 1)
                  reinterpret_cast<float*>(p.out)[idx] = a4[t];
                else if (p.out_dtype == 2)
                  reinterpret_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(a4[t]);
                else
                  reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn(a4[t]);
              }
            }
          }
        }
      } else {
        // D^T output: consecutive threads take consecutive rows, which are contiguous in memory
#pragma unroll 4
        for (int e = et; e < R * TILE_Q; e += kEpiThreads) {
          const int lrow = e % R, col = e / R, g = col >> 2;
          const int off = ((g / kPieces) * R + lrow) * CW + (((g % kPieces) ^ (lrow & (kPieces - 1))) << 2) + (col & 3);
          float acc = 0.f;
          for (int src = 0; src < S; ++src) acc += recv[src * (R * TILE_Q) + off];
          emit(acc, tp * kTileP + crank * R + lrow, tq * TILE_Q + col);
        }
      }
    }
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
}

}  // namespace b200

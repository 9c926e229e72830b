// Host side of libb200_gemm.so: argument validation, plan resolution, TMA tensor-map encoding, variant table
// and launch. Exports the C ABI declared in include/b200_gemm.h. No torch types; no device allocation; no sync.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/b200_gemm.h"
#include "aux_kernels.cuh"
#include "variants.h"

namespace b200 {

constexpr int kMaxDevices = 16;
constexpr uint64_t kCounterBytes = 1u << 20;  // fixed ticket region at the start of the workspace (262144 tiles)

// ------------------------------------------------------------------ driver entry point (no -lcuda link needed)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

static GetAddressRangeFn get_address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GetAddressRangeFn>(ptr);
  });
  return fn;
}

static thread_local char g_last_cuda_error[256] = "";

// ------------------------------------------------------------------ variant table
// The kernels themselves are instantiated in variants_*.cu; this is the menu: (tile_n, CTAs per tile, K elements per
// stage, deepest ring). The first entry of a (tile, cta_group) is the default when the policy leaves tile_k at 0.
struct Variant {
  int tile_q, cta_group, tile_k, max_stages;
};
static const Variant kVariants[] = {
    {16, 1, 128, 5}, {32, 1, 128, 5}, {64, 1, 128, 4}, {128, 1, 128, 3}, {256, 1, 64, 4}, {128, 2, 64, 8},
    {256, 2, 64, 6}, {192, 2, 64, 6}, {16, 1, 64, 8},  {32, 1, 64, 8},   {64, 1, 64, 8},  {128, 1, 64, 6},
    {512, 2, 64, 4},
};
constexpr int kNumVariants = sizeof(kVariants) / sizeof(kVariants[0]);
constexpr int kMaxStages = 12;

static KernelFn variant_fn(const Variant& v, int stages) {
  if (v.cta_group == 2) return pair_variant(v.tile_q, stages);
  return v.tile_k == 128 ? single_k128_variant(v.tile_q, stages) : single_k64_variant(v.tile_q, stages);
}

// The 512-column pair variant takes the width of its tiles at run time: any multiple of 32 above 256.
static int variant_width(int tile_n, int cta_group) {
  return (cta_group == 2 && tile_n > 256 && tile_n <= 512 && tile_n % 32 == 0) ? 512 : tile_n;
}

static const Variant* find_variant(int tile_q, int cta_group, int tile_k) {
  tile_q = variant_width(tile_q, cta_group);
  for (int i = 0; i < kNumVariants; ++i)
    if (kVariants[i].tile_q == tile_q && kVariants[i].cta_group == cta_group &&
        (tile_k == 0 || kVariants[i].tile_k == tile_k))
      return &kVariants[i];
  return nullptr;
}

// V rows of one CTA as laid out in a stage: whole 64-row boxes once there are more than 64 (96 -> 128)
static int v_slot_rows(int tile_q, int cta_group) {
  const int rows = tile_q / cta_group;
  return rows > 64 ? (rows + 63) / 64 * 64 : rows;
}

static int dyn_smem_bytes(int tile_q, int stages, int cta_group, int tile_k) {
  const int staging0 = tile_q >= 64 ? 4 * 2 * 32 * 128 : 0;
  const int recv = tile_q <= 64 ? kTileP * tile_q * 4 : 0;
  const int staging = recv > staging0 ? recv : staging0;
  const int bias = tile_q > 256 ? tile_q * 2 : 256 * 4;
  return stages * (kTileP * tile_k * 2 + v_slot_rows(tile_q, cta_group) * tile_k * 2) + staging + bias + (2 * stages + 4) * 8 + 32 + 1024;
}

struct DeviceInfo {
  int sm_count = 0;
  bool attr_set[kNumVariants][kMaxStages + 1][2] = {};  // [variant][stages][with loader warps]
};
static DeviceInfo g_dev[kMaxDevices];
static std::mutex g_dev_mutex;

static int current_device_info(DeviceInfo** out, int* dev_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_GEMM_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceInfo& d = g_dev[dev];
  if (d.sm_count == 0) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || d.sm_count <= 0)
      return B200_GEMM_ERR_LAUNCH;
  }
  *out = &d;
  *dev_out = dev;
  return 0;
}

// ------------------------------------------------------------------ plan
static inline uint64_t round_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

static bool tma_encodable(const void* ptr, int64_t ld) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && ((ld * 2) & 15) == 0;
}
// A K-contiguous operand whose rows start on 8-byte boundaries can be fetched by the loader warps (cp.async, 8 or 16
// bytes per copy) when TMA cannot describe it.
static bool loader_fetchable(const void* ptr, int64_t ld, int mn_major) {
  return !mn_major && (reinterpret_cast<uintptr_t>(ptr) & 7) == 0 && ((ld * 2) & 7) == 0;
}

struct Resolved {
  b200_gemm_plan plan;
  // operand roles after swap
  const void* u_ptr;
  const void* v_ptr;
  int64_t u_ld, v_ld;
  int u_mn, v_mn;  // 1 = MN-major (P/Q contiguous)
  int P, Q;
  uint64_t off_partials, off_repack_a, off_repack_b;
  int64_t ra_ld, rb_ld;  // pitches of the repacked images
};

static int resolve(const b200_gemm_args* a, Resolved* r, bool need_sm_count, int sm_count_hint) {
  if (a == nullptr) return B200_GEMM_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return B200_GEMM_ERR_BAD_ARG;
  if (a->m > 0x7fffffffLL || a->n > 0x7fffffffLL || a->k > 0x7fffffffLL) return B200_GEMM_ERR_TOO_LARGE;
  if (a->in_dtype != B200_GEMM_DTYPE_BF16 && a->in_dtype != B200_GEMM_DTYPE_FP16) return B200_GEMM_ERR_BAD_ARG;
  if (a->out_dtype != a->in_dtype && a->out_dtype != B200_GEMM_DTYPE_FP32) return B200_GEMM_ERR_BAD_ARG;
  const int64_t a_min_ld = a->a_trans ? a->m : a->k;
  const int64_t b_min_ld = a->b_trans ? a->k : a->n;
  if (a->lda < a_min_ld || a->ldb < b_min_ld || a->ldo < a->n) return B200_GEMM_ERR_BAD_ARG;

  const b200_gemm_policy& pol = a->policy;
  b200_gemm_plan& pl = r->plan;
  memset(&pl, 0, sizeof(pl));
  pl.cta_group = pol.cta_group == 0 ? 1 : pol.cta_group;
  if (pl.cta_group != 1 && pl.cta_group != 2) return B200_GEMM_ERR_BAD_POLICY;
  pl.swap_ab = pol.swap_ab ? 1 : 0;
  pl.tile_m = kTileP * pl.cta_group;
  pl.tile_n = pol.tile_n;
  pl.group_m = pol.group_m < 0 ? 0 : pol.group_m;
  const Variant* var = find_variant(pl.tile_n, pl.cta_group, pol.tile_k);
  if (var == nullptr) return B200_GEMM_ERR_BAD_POLICY;
  pl.tile_k = var->tile_k;

  // A is K-major when 'n'; B[K,N] is K-major when 't'.
  const int a_mn = a->a_trans ? 1 : 0;
  const int b_mn = a->b_trans ? 0 : 1;
  // Operands TMA cannot describe are copied into an aligned image first; when the policy asks for it and their layout
  // allows, the kernel's loader warps fetch them instead (no copy, no scratch, but far slower: see b200_gemm.h).
  const bool loader_ok = pol.loader != 0 && loader_variant(pl.tile_n, pl.cta_group, var->tile_k, nullptr) != nullptr;
  pl.a_loader = (!tma_encodable(a->a, a->lda) && loader_ok && loader_fetchable(a->a, a->lda, a_mn)) ? 1 : 0;
  pl.b_loader = (!tma_encodable(a->b, a->ldb) && loader_ok && loader_fetchable(a->b, a->ldb, b_mn)) ? 1 : 0;
  pl.a_repacked = (tma_encodable(a->a, a->lda) || pl.a_loader) ? 0 : 1;
  pl.b_repacked = (tma_encodable(a->b, a->ldb) || pl.b_loader) ? 0 : 1;
  // Repacked images: K-major operand -> [rows, round_up(K,8)]; MN-major operand -> [K, round_up(rows,8)].
  const int64_t a_rows = a_mn ? a->k : a->m, a_cols = a_mn ? a->m : a->k;
  const int64_t b_rows = b_mn ? a->k : a->n, b_cols = b_mn ? a->n : a->k;
  r->ra_ld = (int64_t)round_up(a_cols, 8);
  r->rb_ld = (int64_t)round_up(b_cols, 8);

  if (!pl.swap_ab) {
    r->P = (int)a->m, r->Q = (int)a->n;
    r->u_mn = a_mn, r->v_mn = b_mn;
  } else {
    r->P = (int)a->n, r->Q = (int)a->m;
    r->u_mn = b_mn, r->v_mn = a_mn;
  }
  // an MN-major operand is fetched in boxes 64 elements wide: each CTA's share of tile_n must be at least one box (a
  // share of 96 columns takes two boxes and uses one and a half)
  if (r->v_mn && var->tile_q / pl.cta_group < 64) return B200_GEMM_ERR_BAD_POLICY;

  pl.tiles_p = (r->P + pl.tile_m - 1) / pl.tile_m;
  pl.tiles_q = (r->Q + pl.tile_n - 1) / pl.tile_n;
  const int64_t tiles = (int64_t)pl.tiles_p * pl.tiles_q;
  const int kb_total = (int)((a->k + pl.tile_k - 1) / pl.tile_k);
  pl.split_k = pol.split_k <= 0 ? 1 : pol.split_k;
  if (pl.split_k > kb_total) pl.split_k = kb_total;  // never an empty slice
  if (tiles * pl.split_k > 0x7fffffffLL) return B200_GEMM_ERR_TOO_LARGE;
  pl.num_units = (int)(tiles * pl.split_k);

  int stages = pol.stages;
  if (stages <= 0 || stages > var->max_stages) stages = var->max_stages;
  while (stages >= 2 && variant_fn(*var, stages) == nullptr) --stages;
  if (stages < 2) return B200_GEMM_ERR_BAD_POLICY;
  if (pl.a_loader || pl.b_loader) loader_variant(pl.tile_n, pl.cta_group, var->tile_k, &stages);  // one depth is built
  pl.stages = stages;
  pl.smem_bytes = dyn_smem_bytes(var->tile_q, stages, pl.cta_group, pl.tile_k);
  pl.tmem_cols = 32;
  while (pl.tmem_cols < 2 * var->tile_q && pl.tmem_cols < 512) pl.tmem_cols *= 2;  // powers of two; a 512-column variant has one accumulator

  int sms = sm_count_hint;
  if (need_sm_count && sms <= 0) return B200_GEMM_ERR_LAUNCH;
  if (sms <= 0) sms = 148;
  // `cap` counts schedulable walkers: CTAs, or CTA pairs when two CTAs share a tile.
  int cap = (pol.max_ctas > 0 ? pol.max_ctas : sms) / pl.cta_group;
  if (cap < 1) cap = 1;
  pl.grid = (pl.num_units < cap ? pl.num_units : cap) * pl.cta_group;

  // Stream-K: tiles that do not fill a whole wave of `cap` CTAs are cut into equal contiguous K spans, one per
  // CTA; whole waves stay data-parallel. A remainder that would give spans shorter than half a tile (many
  // contributors per tile) borrows one full wave; with less than one wave of tiles, spans shorter than kMinSpan K
  // blocks are not worth a pipeline fill and fewer CTAs are used.
  pl.stream_k = 0, pl.sk_tiles = 0, pl.sk_slots = 0;
  if (pol.stream_k && tiles <= 0x7fffffffLL) {
    constexpr int64_t kMinSpan = 4;
    int64_t g = cap;
    int64_t sk = tiles % g;
    if (tiles < g) sk = tiles;
    const int64_t borrow_below = kb_total / 2 > kMinSpan ? kb_total / 2 : kMinSpan;
    if (sk > 0 && tiles > g && sk * kb_total / g < borrow_below) {
      sk += g;  // spans of at least one tile: at most three contributors per cut tile
    } else if (sk > 0 && sk * kb_total / g < kMinSpan) {
      g = sk * kb_total / kMinSpan;
      if (g > cap) g = cap;
    }
    if (sk > 0 && g >= 1 && sk * kb_total / g >= kMinSpan && sk * kb_total >= g) {
      const int64_t span_min = sk * kb_total / g;
      pl.stream_k = 1;
      pl.split_k = 1;
      pl.num_units = (int)tiles;
      pl.sk_tiles = (int)sk;
      pl.sk_slots = (int)((kb_total + span_min - 1) / span_min + 1);
      pl.grid = (int)g * pl.cta_group;
    } else if (sk == 0) {
      pl.split_k = 1;  // whole waves only: plain data-parallel
      pl.num_units = (int)tiles;
      pl.grid = (int)(tiles < cap ? tiles : cap) * pl.cta_group;
    }
  }

  // Cluster split-K: the K slices of a tile are the CTAs of one thread-block cluster and reduce through distributed
  // shared memory: no workspace, no tickets. One tile per cluster, so the grid is not persistent.
  pl.cluster_split = 0;
  if (pol.split_mode == B200_GEMM_SPLIT_CLUSTER && pl.split_k > 1 && !pl.stream_k) {
    if (pl.cta_group != 1) return B200_GEMM_ERR_BAD_POLICY;
    int s = 16;
    while (s > pl.split_k) s >>= 1;  // largest power of two <= split_k (split_k was clamped to the K blocks)
    pl.split_k = s;
    pl.num_units = (int)(tiles * s);
    pl.grid = pl.num_units;
    pl.cluster_split = s > 1 ? s : 0;
    // Tiles wider than 64 receive the cluster's rows (128 x tile_n floats) in the operand ring: it must be that large.
    if (pl.cluster_split && pl.tile_n > 64 &&
        pl.stages * (kTileP * pl.tile_k * 2 + pl.tile_n * pl.tile_k * 2) < kTileP * pl.tile_n * 4)
      return B200_GEMM_ERR_BAD_POLICY;
  }
  // Atomic mode: K-parallel units add their fp32 sums straight into C with TMA reduce-add. Needs an fp32 C that TMA can
  // reach (16-byte aligned rows, a whole number of 4-column groups), tiles at least 64 wide and C written untransposed;
  // where that does not hold the ticket mode is used instead (plan.atomic_out tells which).
  const bool k_parallel = (pl.split_k > 1 && pl.cluster_split == 0) || pl.sk_tiles > 0;
  pl.atomic_out = (pol.split_mode == B200_GEMM_SPLIT_ATOMIC && k_parallel && a->out_dtype == B200_GEMM_DTYPE_FP32 &&
                   !pl.swap_ab && pl.tile_n >= 64 && (reinterpret_cast<uintptr_t>(a->out) & 15) == 0 && (a->ldo & 3) == 0 &&
                   (a->n & 3) == 0)
                      ? 1
                      : 0;
  const bool tickets = k_parallel && !pl.atomic_out;
  if (tickets && tiles * pl.cta_group > (int64_t)(kCounterBytes / 4)) return B200_GEMM_ERR_TOO_LARGE;
  // The ticket region has a fixed size and is reserved by every call that uses the workspace at all, so that no call
  // ever writes partial sums or a repack image where another call keeps its tickets.
  pl.counter_bytes = (tickets || pl.a_repacked || pl.b_repacked) ? kCounterBytes : 0;
  pl.partial_bytes = pl.atomic_out   ? 0
                     : pl.sk_tiles > 0 ? (uint64_t)pl.sk_tiles * pl.sk_slots * pl.tile_m * var->tile_q * 4
                     : (pl.split_k > 1 && pl.cluster_split == 0) ? (uint64_t)pl.num_units * pl.tile_m * var->tile_q * 4
                                                                 : 0;
  const uint64_t ra = pl.a_repacked ? round_up((uint64_t)a_rows * r->ra_ld * 2, 256) : 0;
  const uint64_t rb = pl.b_repacked ? round_up((uint64_t)b_rows * r->rb_ld * 2, 256) : 0;
  pl.repack_bytes = ra + rb;
  r->off_partials = pl.counter_bytes;
  r->off_repack_a = r->off_partials + pl.partial_bytes;
  r->off_repack_b = r->off_repack_a + ra;
  pl.workspace_bytes = r->off_repack_b + rb;
  return 0;
}

// ------------------------------------------------------------------ tensor maps
// K-major operand [rows, K] (K contiguous): dims {K, rows}, box {64, box_rows}.
// MN-major operand [K, rows] (rows contiguous): dims {rows, K}, box {64, 64}.
static int encode_operand(CUtensorMap* map, const void* ptr, int in_dtype, int mn_major, int64_t rows, int64_t k,
                          int64_t ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return B200_GEMM_ERR_DRIVER;
  const CUtensorMapDataType dt = in_dtype == B200_GEMM_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[2], strides[1];
  cuuint32_t box[2], estr[2] = {1, 1};
  if (!mn_major) {
    dims[0] = (cuuint64_t)k, dims[1] = (cuuint64_t)rows;
    box[0] = kBoxK, box[1] = (cuuint32_t)box_rows;
  } else {
    dims[0] = (cuuint64_t)rows, dims[1] = (cuuint64_t)k;
    box[0] = 64, box[1] = kBoxK;
  }
  strides[0] = (cuuint64_t)ld * 2;
  const CUresult res = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return res == CUDA_SUCCESS ? 0 : B200_GEMM_ERR_TENSOR_MAP;
}

// smem matrix descriptor template (everything but the start address) for a 128-byte-swizzled operand stage.
//   bits 16-29 leading byte offset >> 4, 32-45 stride byte offset >> 4, 46-47 version (1), 61-63 layout (2 = SW128).
// K-major: rows are 128 B apart, 8-row groups 1024 B apart (SBO); LBO unused (1). K=16 step = 32 B.
// MN-major: each 64-element box is [64 K rows x 128 B]; 8-K-row groups 1024 B apart (SBO), boxes 8192 B apart (LBO);
//           K=16 step = 2048 B.
static void make_desc(int mn_major, uint32_t* hi, uint32_t* lo, uint32_t* kstep) {
  const uint32_t sbo = 1024 >> 4;
  const uint32_t lbo = mn_major ? (8192 >> 4) : 1;
  *lo = lbo << 16;
  *hi = sbo | (1u << 14) | (2u << 29);
  *kstep = mn_major ? (2048 >> 4) : (32 >> 4);
}

static uint32_t make_idesc(int in_dtype, int u_mn, int v_mn, int mma_m, int mma_n) {
  const uint32_t fmt = in_dtype == B200_GEMM_DTYPE_BF16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(u_mn) << 15) | (uint32_t(v_mn) << 16) | (uint32_t(mma_n >> 3) << 17) |
         (uint32_t(mma_m >> 4) << 24);
}

static int set_cuda_error(cudaError_t e) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s", cudaGetErrorString(e));
  return B200_GEMM_ERR_LAUNCH;
}

// A fully resolved call: everything the launch needs, so that repeating it costs one kernel launch (two when an operand must be repacked first)
// and no host-side planning or tensor-map encoding.
struct RepackJob {
  const uint16_t* src;
  uint16_t* dst;
  long long src_ld, dst_ld;
  int rows, cols, blocks;
};

}  // namespace b200

struct b200_gemm_handle {
  b200::GemmParams params;
  b200::KernelFn fn;
  int grid, threads, smem_bytes, device, cta_group, cluster_split, pdl;
  int n_repack;
  b200::RepackJob repack[2];
  int init_out;  // atomic split mode: C is set to the bias (or zero) by a small kernel before the GEMM
  int m, n, bias_dtype;
  b200_gemm_plan plan;
};

namespace b200 {

static int prepare(const b200_gemm_args* a, b200_gemm_handle* h) {
  DeviceInfo* dev = nullptr;
  int dev_id = 0;
  int rc = current_device_info(&dev, &dev_id);
  if (rc) return rc;
  Resolved r;
  rc = resolve(a, &r, true, dev->sm_count);
  if (rc) return rc;
  const b200_gemm_plan& pl = r.plan;
  if (a->a == nullptr || a->b == nullptr || a->out == nullptr) return B200_GEMM_ERR_BAD_ARG;
  if (pl.workspace_bytes > 0 && (a->workspace == nullptr || a->workspace_bytes < pl.workspace_bytes ||
                                 (reinterpret_cast<uintptr_t>(a->workspace) & 255) != 0))
    return B200_GEMM_ERR_WORKSPACE;
  uint8_t* ws = reinterpret_cast<uint8_t*>(a->workspace);
  h->plan = pl;
  h->device = dev_id;
  h->n_repack = 0;

  // Operands TMA cannot describe are first copied into an aligned image (same stream, ordered before the GEMM).
  const void* pa = a->a;
  const void* pb = a->b;
  int64_t lda = a->lda, ldb = a->ldb;
  const int a_mn = a->a_trans ? 1 : 0, b_mn = a->b_trans ? 0 : 1;
  auto add_repack = [&](const void* src, int64_t src_ld, uint64_t off, int64_t dst_ld, int rows, int cols) {
    RepackJob& j = h->repack[h->n_repack++];
    j.src = reinterpret_cast<const uint16_t*>(src);
    j.dst = reinterpret_cast<uint16_t*>(ws + off);
    j.src_ld = src_ld, j.dst_ld = dst_ld, j.rows = rows, j.cols = cols;
    const long long total = (long long)rows * ((cols + 7) / 8);
    const long long want = (total + 255) / 256;
    j.blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    return j.dst;
  };
  if (pl.a_repacked) {
    pa = add_repack(a->a, a->lda, r.off_repack_a, r.ra_ld, (int)(a_mn ? a->k : a->m), (int)(a_mn ? a->m : a->k));
    lda = r.ra_ld;
  }
  if (pl.b_repacked) {
    pb = add_repack(a->b, a->ldb, r.off_repack_b, r.rb_ld, (int)(b_mn ? a->k : a->n), (int)(b_mn ? a->n : a->k));
    ldb = r.rb_ld;
  }

  GemmParams& p = h->params;
  memset(&p, 0, sizeof(p));
  const int mma_n = pl.tile_n > 256 ? 256 : pl.tile_n;  // columns of one tcgen05.mma (a 512-wide tile issues two per K step)
  const void* u_ptr = pl.swap_ab ? pb : pa;
  const void* v_ptr = pl.swap_ab ? pa : pb;
  const int64_t u_ld = pl.swap_ab ? ldb : lda, v_ld = pl.swap_ab ? lda : ldb;
  const int u_cp = pl.swap_ab ? pl.b_loader : pl.a_loader, v_cp = pl.swap_ab ? pl.a_loader : pl.b_loader;
  if (!u_cp) {
    rc = encode_operand(&p.tmap_u, u_ptr, a->in_dtype, r.u_mn, r.P, a->k, u_ld, kTileP);
    if (rc) return rc;
  }
  if (!v_cp) {
    rc = encode_operand(&p.tmap_v, v_ptr, a->in_dtype, r.v_mn, r.Q, a->k, v_ld, mma_n / pl.cta_group);
    if (rc) return rc;
  }
  p.u_cp = u_cp, p.v_cp = v_cp;
  p.u_src = u_ptr, p.v_src = v_ptr;
  p.u_pitch = u_ld * 2, p.v_pitch = v_ld * 2;
  const int v_tma_rows = r.v_mn ? v_slot_rows(pl.tile_n, pl.cta_group) : pl.tile_n / pl.cta_group;  // whole boxes when MN-major
  p.tma_tx_bytes = (uint32_t)(pl.cta_group * pl.tile_k * 2 * ((u_cp ? 0 : kTileP) + (v_cp ? 0 : v_tma_rows)));
  p.out = a->out;
  p.bias = a->bias;
  {
    // Finished tiles leave through TMA stores when C's rows are 16-byte aligned (and D is not written transposed).
    const int es = a->out_dtype == B200_GEMM_DTYPE_FP32 ? 4 : 2;
    p.tma_store = 0;
    if (!pl.swap_ab && pl.tile_n >= 64 && (reinterpret_cast<uintptr_t>(a->out) & 15) == 0 && ((a->ldo * es) & 15) == 0) {
      EncodeTiledFn enc = get_encode_fn();
      if (enc == nullptr) return B200_GEMM_ERR_DRIVER;
      const CUtensorMapDataType dt = a->out_dtype == B200_GEMM_DTYPE_FP32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : a->out_dtype == B200_GEMM_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      cuuint64_t dims[2] = {(cuuint64_t)a->n, (cuuint64_t)a->m};
      cuuint64_t strides[1] = {(cuuint64_t)a->ldo * es};
      cuuint32_t box[2] = {(cuuint32_t)(128 / es), 32};
      cuuint32_t estr[2] = {1, 1};
      if (enc(&p.tmap_out, dt, 2, a->out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
        p.tma_store = 1;
    }
  }
  p.atomic_out = pl.atomic_out;
  if (pl.atomic_out && !p.tma_store) return B200_GEMM_ERR_TENSOR_MAP;
  h->init_out = pl.atomic_out;
  h->m = (int)a->m, h->n = (int)a->n, h->bias_dtype = a->in_dtype;
  p.tickets = reinterpret_cast<int*>(ws);
  p.partials = reinterpret_cast<float*>(ws + r.off_partials);
  p.status = a->status;
  const uint64_t trace_need = (uint64_t)pl.grid * kTraceRoles * kTraceItems * kTraceStamps;
  p.trace = (a->trace != nullptr && a->trace_words >= trace_need) ? reinterpret_cast<unsigned long long*>(a->trace) : nullptr;
  p.trace_detail = (p.trace != nullptr && a->trace_words >= 2 * trace_need) ? 1 : 0;
  p.ldo = a->ldo;
  p.P = r.P, p.Q = r.Q, p.K = (int)a->k;
  p.tiles_p = pl.tiles_p, p.tiles_q = pl.tiles_q, p.num_tiles = pl.tiles_p * pl.tiles_q;
  p.kb_total = (int)((a->k + pl.tile_k - 1) / pl.tile_k);
  p.split_k = pl.split_k;
  p.cluster_split = pl.cluster_split;
  p.num_units = pl.num_units;
  p.sk_tiles = pl.sk_tiles;
  p.sk_slots = pl.sk_slots;
  p.group_p = pl.group_m;
  p.swap_out = pl.swap_ab;
  p.out_dtype = a->out_dtype;
  p.in_dtype = a->in_dtype;
  p.u_mn_major = r.u_mn, p.v_mn_major = r.v_mn;
  p.idesc = make_idesc(a->in_dtype, r.u_mn, r.v_mn, pl.tile_m, mma_n);
  p.idesc2 = pl.tile_n > 256 ? make_idesc(a->in_dtype, r.u_mn, r.v_mn, pl.tile_m, pl.tile_n - 256) : 0;
  p.tile_q = pl.tile_n;
  make_desc(r.u_mn, &p.u_desc_hi, &p.u_desc_lo, &p.u_kstep);
  make_desc(r.v_mn, &p.v_desc_hi, &p.v_desc_lo, &p.v_kstep);
  p.wait_limit_ns = a->policy.wait_limit_us > 0 ? (unsigned long long)a->policy.wait_limit_us * 1000ull : kWaitLimitNs;

  const Variant* var = find_variant(pl.tile_n, pl.cta_group, pl.tile_k);
  const int vi = (int)(var - kVariants);
  const int with_loader = (u_cp || v_cp) ? 1 : 0;
  h->fn = with_loader ? loader_variant(pl.tile_n, pl.cta_group, pl.tile_k, nullptr) : variant_fn(*var, pl.stages);
  if (h->fn == nullptr) return B200_GEMM_ERR_BAD_POLICY;
  h->threads = with_loader ? kThreadsLoader : kThreads;
  h->grid = pl.grid;
  h->smem_bytes = pl.smem_bytes;
  h->cta_group = pl.cta_group;
  h->cluster_split = pl.cluster_split;
  h->pdl = a->policy.no_pdl ? 0 : 1;
  if (pl.cluster_split > 8) {
    // clusters of 16 CTAs are outside the portable range: the kernel has to opt in
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(h->fn), cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return set_cuda_error(e);
  }
  {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (!dev->attr_set[vi][pl.stages][with_loader]) {
      cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(h->fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           pl.smem_bytes);
      if (e != cudaSuccess) return set_cuda_error(e);
      dev->attr_set[vi][pl.stages][with_loader] = true;
    }
  }
  return 0;
}

static int run(const b200_gemm_handle* h, cudaStream_t stream) {
  if (h->n_repack > 0) {  // one launch for both operands when both need it
    const RepackJob& j0 = h->repack[0];
    const RepackJob j1 = h->n_repack > 1 ? h->repack[1] : RepackJob{nullptr, nullptr, 0, 0, 0, 0, 0};
    repack_rows_kernel<<<j0.blocks + j1.blocks, 256, 0, stream>>>(j0.src, j0.src_ld, j0.dst, j0.dst_ld, j0.rows, j0.cols, j0.blocks,
                                                                  j1.src, j1.src_ld, j1.dst, j1.dst_ld, j1.rows, j1.cols);
    cudaError_t re = cudaGetLastError();
    if (re != cudaSuccess) return set_cuda_error(re);
  }
  if (h->init_out) {
    const long long total4 = (long long)h->m * (h->n / 4);
    const long long want = (total4 + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    init_out_rows_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<float*>(h->params.out), h->params.ldo, h->m, h->n,
                                                     h->params.bias, h->bias_dtype);
    cudaError_t ie = cudaGetLastError();
    if (ie != cudaSuccess) return set_cuda_error(ie);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(h->grid, 1, 1);
  cfg.blockDim = dim3(h->threads, 1, 1);
  cfg.dynamicSmemBytes = h->smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (h->cta_group == 2 || h->cluster_split > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = h->cta_group == 2 ? 2 : h->cluster_split;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (h->pdl) {
    // the kernel's set-up phase may overlap the previous kernel of this stream; it waits before touching memory
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = n_attr ? attr : nullptr;
  cfg.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, h->fn, h->params);
  if (e != cudaSuccess) return set_cuda_error(e);
  return 0;
}

// ------------------------------------------------------------------ built-in scratch for callers that cannot allocate
// Lives in every GPU that loads this library, for the life of the process. In host code the name below is only a
// stand-in for the device symbol; its device address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[B200_GEMM_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_ptr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

static int static_scratch_for_current_device(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_GEMM_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess) return set_cuda_error(e);
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0) return B200_GEMM_ERR_WORKSPACE;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}

}  // namespace b200

extern "C" {

int b200_gemm_a16w16_static_scratch(const b200_gemm_args* args, void* cuda_stream) {
  if (args == nullptr) return B200_GEMM_ERR_BAD_ARG;
  b200_gemm_plan plan;
  int rc = b200_gemm_plan_query(args, &plan);
  if (rc) return rc;
  b200_gemm_args local = *args;
  if (plan.workspace_bytes > (uint64_t)B200_GEMM_STATIC_SCRATCH_BYTES && (plan.a_repacked || plan.b_repacked) && !local.policy.loader) {
    // The aligned copies of the operands do not fit the built-in array: let the kernel's loader warps fetch them
    // where their layout allows (slower, but needs no scratch for them).
    local.policy.loader = 1;
    rc = b200_gemm_plan_query(&local, &plan);
    if (rc) return rc;
  }
  if (plan.workspace_bytes > (uint64_t)B200_GEMM_STATIC_SCRATCH_BYTES) return B200_GEMM_ERR_TOO_LARGE;
  local.workspace = nullptr;
  local.workspace_bytes = 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  if (plan.workspace_bytes > 0) {
    void* scratch = nullptr;
    rc = b200::static_scratch_for_current_device(&scratch);
    if (rc) return rc;
    local.workspace = scratch;
    local.workspace_bytes = B200_GEMM_STATIC_SCRATCH_BYTES;
    // The array keeps whatever the previous call left. Partial sums and repack images are fully rewritten before
    // they are read; the tickets must start at zero, so the ones this call uses are cleared first (same stream).
    if (plan.split_k > 1 || plan.sk_tiles > 0) {
      const size_t ticket_bytes = (size_t)plan.tiles_p * plan.tiles_q * plan.cta_group * sizeof(int);
      cudaError_t e = cudaMemsetAsync(scratch, 0, ticket_bytes, stream);
      if (e != cudaSuccess) return b200::set_cuda_error(e);
    }
  }
  b200_gemm_handle h;
  rc = b200::prepare(&local, &h);
  if (rc) return rc;
  return b200::run(&h, stream);
}

int b200_gemm_selftest(void* cuda_stream, int32_t* failed_case) {
  // Scratch map (bytes from the start of the built-in array): GEMM workspace | A | B | bias | out | reference | counters.
  constexpr size_t kWs = 0, kWsBytes = 8u << 20, kA = kWsBytes, kB = kA + (512u << 10), kBias = kB + (512u << 10),
                   kOut = kBias + (64u << 10), kRef = kOut + (512u << 10), kFlag = kRef + (512u << 10);
  static_assert(kFlag + 256 <= (size_t)B200_GEMM_STATIC_SCRATCH_BYTES, "self-test scratch map");
  constexpr int M = 200, N = 264, K = 328;  // ragged against every tile; all pitches are multiples of 16 bytes
  struct Case {
    int tile_n, cta_group, split_k, split_mode, stream_k, swap_ab, tile_k, fp32_out, bias, k_major_only;
  };
  static const Case cases[] = {
      {64, 1, 1, 0, 0, 0, 0, 0, 1, 0},  {128, 1, 1, 0, 0, 0, 0, 1, 0, 0},  {256, 1, 1, 0, 0, 0, 0, 0, 1, 0},
      {128, 2, 1, 0, 0, 0, 0, 0, 1, 0}, {256, 2, 1, 0, 0, 0, 0, 1, 1, 0},  {128, 1, 1, 0, 0, 0, 64, 0, 0, 0},
      {64, 1, 3, 0, 0, 0, 0, 1, 1, 0},  {64, 1, 2, 2, 0, 0, 0, 0, 1, 0},   {128, 1, 1, 0, 1, 0, 0, 0, 1, 0},
      {16, 1, 1, 0, 0, 0, 0, 0, 1, 1},  {32, 1, 2, 2, 0, 0, 64, 1, 0, 1},  {16, 1, 4, 2, 0, 1, 0, 1, 1, 1},
      {192, 2, 1, 0, 0, 0, 0, 0, 1, 1}, {512, 2, 1, 0, 0, 0, 0, 0, 1, 0},  {512, 2, 2, 0, 0, 0, 0, 1, 1, 0},
      {352, 2, 1, 0, 0, 0, 0, 0, 1, 0},
  };
  if (failed_case) *failed_case = -1;
  void* scratch_v = nullptr;
  int rc = b200::static_scratch_for_current_device(&scratch_v);
  if (rc) return rc;
  unsigned char* scratch = static_cast<unsigned char*>(scratch_v);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  int* flag = reinterpret_cast<int*>(scratch + kFlag);
  int index = 0;
  for (int dtype = 2; dtype <= 3; ++dtype) {
    for (int layout = 0; layout < 4; ++layout) {
      const int a_trans = layout >> 1, b_trans = layout & 1;
      uint16_t* a = reinterpret_cast<uint16_t*>(scratch + kA);
      uint16_t* b = reinterpret_cast<uint16_t*>(scratch + kB);
      uint16_t* bias = reinterpret_cast<uint16_t*>(scratch + kBias);
      const int a_rows = a_trans ? K : M, a_cols = a_trans ? M : K;
      const int b_rows = b_trans ? N : K, b_cols = b_trans ? K : N;
      b200::selftest_fill_kernel<<<64, 256, 0, stream>>>(a, a_rows, a_cols, a_cols, dtype, 1 + layout);
      b200::selftest_fill_kernel<<<64, 256, 0, stream>>>(b, b_rows, b_cols, b_cols, dtype, 2 + dtype);
      b200::selftest_fill_kernel<<<1, 256, 0, stream>>>(bias, 1, N, N, dtype, 3);
      for (int with_bias = 0; with_bias < 2; ++with_bias)
        b200::selftest_ref_kernel<<<128, 256, 0, stream>>>(a, a_cols, a_trans, b, b_cols, b_trans, with_bias ? bias : nullptr, M,
                                                           N, K, dtype,
                                                           reinterpret_cast<float*>(scratch + kRef) + (size_t)with_bias * M * N);
      for (const Case& c : cases) {
        ++index;
        // The operand on the MMA N axis of a tile narrower than 64 must be K-contiguous: B stored [N,K], or A [M,K] after a swap.
        if (c.k_major_only && (c.swap_ab ? a_trans != 0 : b_trans == 0)) continue;
        b200_gemm_args args;
        memset(&args, 0, sizeof(args));
        args.a = a, args.b = b, args.out = scratch + kOut, args.bias = c.bias ? bias : nullptr;
        args.m = M, args.n = N, args.k = K;
        args.lda = a_cols, args.ldb = b_cols, args.ldo = N;
        args.a_trans = a_trans, args.b_trans = b_trans;
        args.in_dtype = dtype, args.out_dtype = c.fp32_out ? B200_GEMM_DTYPE_FP32 : dtype;
        args.policy.tile_n = c.tile_n, args.policy.cta_group = c.cta_group, args.policy.split_k = c.split_k;
        args.policy.split_mode = c.split_mode, args.policy.stream_k = c.stream_k, args.policy.swap_ab = c.swap_ab;
        args.policy.tile_k = c.tile_k;
        args.workspace = scratch + kWs, args.workspace_bytes = kWsBytes;
        cudaError_t e = cudaMemsetAsync(scratch + kWs, 0, B200_GEMM_COUNTER_BYTES, stream);  // tickets start at zero
        if (e == cudaSuccess) e = cudaMemsetAsync(scratch + kOut, 0xff, (size_t)M * N * 4, stream);  // NaN-poison the output
        if (e == cudaSuccess) e = cudaMemsetAsync(flag, 0, sizeof(int), stream);
        if (e != cudaSuccess) return b200::set_cuda_error(e);
        rc = b200_gemm_a16w16(&args, cuda_stream);
        if (rc) {
          if (failed_case) *failed_case = index;
          return rc;
        }
        b200::selftest_compare_kernel<<<64, 256, 0, stream>>>(scratch + kOut, args.out_dtype,
                                                             reinterpret_cast<float*>(scratch + kRef) + (size_t)(c.bias ? 1 : 0) * M * N,
                                                             (long long)M * N, flag);
        int bad = 0;
        e = cudaMemcpyAsync(&bad, flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return b200::set_cuda_error(e);
        if (bad != 0) {
          if (failed_case) *failed_case = index;
          return B200_GEMM_ERR_SELFTEST;
        }
      }
    }
  }
  return B200_GEMM_OK;
}

int b200_gemm_a16w16(const b200_gemm_args* args, void* cuda_stream) {
  b200_gemm_handle h;
  const int rc = b200::prepare(args, &h);
  if (rc) return rc;
  return b200::run(&h, reinterpret_cast<cudaStream_t>(cuda_stream));
}

int b200_gemm_prepare(const b200_gemm_args* args, b200_gemm_handle** out) {
  if (out == nullptr) return B200_GEMM_ERR_BAD_ARG;
  *out = nullptr;
  b200_gemm_handle* h = new (std::nothrow) b200_gemm_handle;
  if (h == nullptr) return B200_GEMM_ERR_BAD_ARG;
  const int rc = b200::prepare(args, h);
  if (rc) {
    delete h;
    return rc;
  }
  *out = h;
  return 0;
}

int b200_gemm_launch(const b200_gemm_handle* handle, void* cuda_stream) {
  if (handle == nullptr) return B200_GEMM_ERR_BAD_ARG;
  return b200::run(handle, reinterpret_cast<cudaStream_t>(cuda_stream));
}

void b200_gemm_release(b200_gemm_handle* handle) { delete handle; }

int b200_gemm_plan_query(const b200_gemm_args* args, b200_gemm_plan* plan) {
  if (plan == nullptr) return B200_GEMM_ERR_BAD_ARG;
  b200::Resolved r;
  int sms = 0;
  {
    b200::DeviceInfo* dev = nullptr;
    int dev_id = 0;
    if (b200::current_device_info(&dev, &dev_id) == 0) sms = dev->sm_count;
  }
  const int rc = b200::resolve(args, &r, false, sms);
  if (rc) return rc;
  *plan = r.plan;
  return 0;
}

uint64_t b200_gemm_workspace_bytes(const b200_gemm_args* args) {
  b200_gemm_plan plan;
  if (b200_gemm_plan_query(args, &plan) != 0) return 0;
  return plan.workspace_bytes;
}

int b200_gemm_num_variants(void) { return b200::kNumVariants; }

int b200_gemm_describe_variant(int index, int32_t* tile_n, int32_t* cta_group, int32_t* max_stages, int32_t* tile_k) {
  if (index < 0 || index >= b200::kNumVariants) return B200_GEMM_ERR_BAD_ARG;
  if (tile_n) *tile_n = b200::kVariants[index].tile_q;
  if (cta_group) *cta_group = b200::kVariants[index].cta_group;
  if (max_stages) *max_stages = b200::kVariants[index].max_stages;
  if (tile_k) *tile_k = b200::kVariants[index].tile_k;
  return 0;
}

int b200_gemm_cast_bias(const float* in, void* out, const void* bias, int64_t rows, int64_t cols, int32_t out_dtype,
                        int32_t bias_dtype, void* cuda_stream) {
  if (in == nullptr || out == nullptr || rows < 0 || cols <= 0 || cols > 0x7fffffffLL) return B200_GEMM_ERR_BAD_ARG;
  if (out_dtype < 1 || out_dtype > 3) return B200_GEMM_ERR_BAD_ARG;
  if (bias != nullptr && bias_dtype != B200_GEMM_DTYPE_BF16 && bias_dtype != B200_GEMM_DTYPE_FP16) return B200_GEMM_ERR_BAD_ARG;
  if (cols % 4 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return B200_GEMM_ERR_BAD_ARG;
  if (rows == 0) return 0;
  const long long total4 = rows * cols / 4;
  const long long want = (total4 + 255) / 256;
  const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
  b200::cast_bias_rows_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(in, out, bias, rows, (int)cols,
                                                                                             out_dtype, bias_dtype);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return b200::set_cuda_error(e);
  return 0;
}

int b200_gemm_reduce_slots(const float* slots, int64_t slot_stride, int32_t n_slots, void* out, const void* bias,
                           int64_t rows, int64_t cols, int32_t out_dtype, int32_t bias_dtype, void* cuda_stream) {
  if (slots == nullptr || out == nullptr || n_slots < 1 || rows < 0 || cols <= 0 || cols > 0x7fffffffLL)
    return B200_GEMM_ERR_BAD_ARG;
  if (out_dtype < 1 || out_dtype > 3) return B200_GEMM_ERR_BAD_ARG;
  if (bias != nullptr && bias_dtype != B200_GEMM_DTYPE_BF16 && bias_dtype != B200_GEMM_DTYPE_FP16) return B200_GEMM_ERR_BAD_ARG;
  if (cols % 4 != 0 || slot_stride % 4 != 0 || (n_slots > 1 && slot_stride < rows * cols) ||
      (reinterpret_cast<uintptr_t>(slots) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return B200_GEMM_ERR_BAD_ARG;
  if (rows == 0) return 0;
  const long long total4 = rows * cols / 4;
  const long long want = (total4 + 255) / 256;
  const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
  b200::reduce_slots_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
      slots, slot_stride, n_slots, out, bias, rows, (int)cols, out_dtype, bias_dtype);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return b200::set_cuda_error(e);
  return 0;
}

int b200_peer_export(const void* ptr, b200_peer_handle* handle) {
  if (ptr == nullptr || handle == nullptr) return B200_GEMM_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == sizeof(handle->ipc), "IPC handle size");
  b200::GetAddressRangeFn range = b200::get_address_range_fn();
  if (range == nullptr) return B200_GEMM_ERR_DRIVER;
  CUdeviceptr base = 0;
  size_t bytes = 0;
  if (range(&base, &bytes, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return B200_GEMM_ERR_BAD_ARG;
  memset(handle, 0, sizeof(*handle));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) return b200::set_cuda_error(e);
  memcpy(handle->ipc, &h, sizeof(h));
  handle->offset = reinterpret_cast<uintptr_t>(ptr) - (uintptr_t)base;
  handle->bytes = bytes - handle->offset;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B200_GEMM_ERR_LAUNCH;
  handle->device = dev;
  return 0;
}

int b200_peer_open(const b200_peer_handle* handle, void** ptr) {
  if (handle == nullptr || ptr == nullptr) return B200_GEMM_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle->ipc, sizeof(h));
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return b200::set_cuda_error(e);
  *ptr = static_cast<char*>(base) + handle->offset;
  return 0;
}

int b200_peer_close(void* ptr, const b200_peer_handle* handle) {
  if (ptr == nullptr || handle == nullptr) return B200_GEMM_ERR_BAD_ARG;
  cudaError_t e = cudaIpcCloseMemHandle(static_cast<char*>(ptr) - handle->offset);
  if (e != cudaSuccess) return b200::set_cuda_error(e);
  return 0;
}

int b200_gemm_wait_selftest(int32_t* status, uint32_t limit_us, void* cuda_stream) {
  if (status == nullptr || limit_us == 0 || limit_us > 1000000u) return B200_GEMM_ERR_BAD_ARG;
  b200::wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(status, (unsigned long long)limit_us * 1000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return b200::set_cuda_error(e);
  return 0;
}

const char* b200_gemm_strerror(int code) {
  switch (code) {
    case B200_GEMM_OK: return "ok";
    case B200_GEMM_ERR_BAD_ARG: return "bad argument (null pointer, size, stride or dtype)";
    case B200_GEMM_ERR_BAD_POLICY: return "unsupported policy (tile_n / cta_group / stages / layout combination)";
    case B200_GEMM_ERR_WORKSPACE: return "workspace missing, misaligned (256 B) or smaller than b200_gemm_workspace_bytes()";
    case B200_GEMM_ERR_TENSOR_MAP: return "cuTensorMapEncodeTiled rejected an operand";
    case B200_GEMM_ERR_LAUNCH: return b200::g_last_cuda_error[0] ? b200::g_last_cuda_error : "CUDA runtime error";
    case B200_GEMM_ERR_DRIVER: return "a CUDA driver entry point (cuTensorMapEncodeTiled, cuMemGetAddressRange) is not available";
    case B200_GEMM_ERR_TOO_LARGE: return "size beyond a fixed limit of this entry point";
    case B200_GEMM_ERR_SELFTEST: return "self-test: a known-answer case gave a wrong result";
    default: return "unknown error code";
  }
}

const char* b200_gemm_version(void) { return "b200_gemm 0.1 sm_100a"; }

}  // extern "C"

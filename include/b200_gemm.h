/* C ABI of the B200 (sm_100a) A16W16 GEMM library, libb200_gemm.so.
 *
 * This is the drop-in boundary for the one hot path of xytpai/flydsl-examples:
 *   C[M,N] = A[M,K] * B[K,N] (+ bias[N]), 16-bit inputs, fp32 accumulation, one cast to the output type.
 * Plain pointers and sizes only; no torch types. Every entry point is re-entrant, never synchronises the
 * device, never throws and never aborts: errors come back as negative codes (b200_gemm_strerror).
 * Entry points allocate no device memory unless their comment says so.
 */
#ifndef B200_GEMM_H_
#define B200_GEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype ids: the reference's GEMM_A16W16_DTYPE_{FP32,BF16,FP16} (kernels/gemm_a16w16_gfx950.py:28-30). */
#define B200_GEMM_DTYPE_FP32 1
#define B200_GEMM_DTYPE_BF16 2
#define B200_GEMM_DTYPE_FP16 3

/* error codes */
#define B200_GEMM_OK 0
#define B200_GEMM_ERR_BAD_ARG (-1)        /* null pointer, bad dtype, negative size ...            */
#define B200_GEMM_ERR_BAD_POLICY (-2)     /* tile / stages / split_k outside the supported menu     */
#define B200_GEMM_ERR_WORKSPACE (-3)      /* workspace missing or smaller than workspace_bytes()    */
#define B200_GEMM_ERR_TENSOR_MAP (-4)     /* cuTensorMapEncodeTiled refused the operand             */
#define B200_GEMM_ERR_LAUNCH (-5)         /* CUDA launch error (cudaGetLastError text via strerror) */
#define B200_GEMM_ERR_DRIVER (-6)         /* driver entry point not found                           */
#define B200_GEMM_ERR_TOO_LARGE (-7)      /* size beyond a stated fixed limit                       */
#define B200_GEMM_ERR_SELFTEST (-8)   /* b200_gemm_selftest: a known-answer case gave a wrong result              */

/* size of the ticket region at the start of a workspace */
#define B200_GEMM_COUNTER_BYTES (1u << 20)

/* split-K reduction modes */
#define B200_GEMM_SPLIT_TICKET 0 /* fp32 partial tiles in the workspace; the last-arriving CTA of a tile sums them in
                                    slice order, adds bias and casts once (deterministic; never waits)            */
#define B200_GEMM_SPLIT_ATOMIC 1  /* fp32 outputs: every K slice (or stream-K span) adds its fp32 tile straight into C
                                     with TMA reduce-add (the additions happen in L2), after a small kernel has set C to
                                     the bias (or zero): no workspace, no tickets, no second pass; the order of the
                                     additions, and so the last bits of the result, vary from run to run. Needs an
                                     fp32 C with 16-byte aligned rows, tile_n >= 64, no swap_ab; otherwise the ticket mode
                                     runs (b200_gemm_plan.atomic_out tells). Takes the place of the reference's atomic
                                     split-K epilogue (kernels/gemm_a16w16_gfx950.py:325-375), in fp32 instead of
                                     packed 16-bit                                                                  */
#define B200_GEMM_SPLIT_CLUSTER 2 /* the K slices of a tile are the CTAs of one thread-block cluster (2, 4, 8 or 16);
                                     each CTA sends its partial rows to the row's owner through distributed shared
                                     memory, a cluster barrier, owners sum in rank order. No workspace, no tickets,
                                     deterministic. cta_group 1; split_k is rounded down to a power of two. Tiles wider
                                     than 64 receive into the idle operand ring (one more cluster barrier)          */

/* Blackwell policy. Replaces the reference's compile-time GemmA16W16Gfx950Param
 * (kernels/gemm_a16w16_gfx950.py:33-61): block_m/n/k, stages, split_k, *_waves, group_m, HTI flag. */
typedef struct b200_gemm_policy {
  int32_t tile_n;     /* columns of one tile: 16, 32, 64, 128 or 256; for CTA pairs also 192 and any multiple of 32 from 288 to
                         512 (one kernel variant, two MMAs per K step into one accumulator that fills TMEM: up to a quarter
                         less operand traffic per flop, but the epilogue no longer overlaps the next tile's main loop; the
                         width is a run-time parameter so that the caller can fill whole waves). Tile M is 128 per CTA; the
                         K extent of a pipeline stage follows from the variant, see b200_gemm_describe_variant      */
  int32_t stages;     /* depth of the TMA->smem ring; 0, or more than fit in 227 KB, = as many as fit              */
  int32_t split_k;    /* >= 1 K-slices per output tile (uneven slices allowed, K tail is zero-filled by TMA)      */
  int32_t group_m;    /* grouped rasterisation: tiles are walked in groups of group_m tile rows; 0 = row-major     */
  int32_t swap_ab;    /* 1: compute C^T = B^T A^T so N sits on the 128-row MMA axis (small-M shapes)               */
  int32_t cta_group;  /* 1, or 2 = a CTA pair shares one 256-row tile (tcgen05 cta_group::2)                       */
  int32_t split_mode; /* B200_GEMM_SPLIT_*                                                                       */
  int32_t max_ctas;   /* persistent grid size cap; 0 = number of SMs                                              */
  int32_t stream_k;   /* 1: tail-wave tiles are cut into K spans so every SM gets equal work                      */
  int32_t no_pdl;     /* 1: launch without programmatic dependent launch. By default the kernel's set-up (barriers,
                         TMEM, descriptor prefetch) may overlap the end of the previous kernel in the stream; it
                         waits for that kernel to complete before it reads or writes global memory               */
  int32_t tile_k;     /* K elements per pipeline stage: 64 or 128 where the variant table has both (single-CTA tiles up
                         to 128 wide); 0 = the tile's default (128 there, 64 for 256-wide tiles and CTA pairs)      */
  int32_t wait_limit_us; /* time limit of every wait inside the kernel, in microseconds; 0 = 2 seconds. A wait that
                            runs out makes the kernel give up, free what it holds and report through `status`       */
  int32_t loader; /* 1: fetch operands TMA cannot describe (base or pitch not a multiple of 16 bytes) inside the GEMM
                     kernel with its cp.async loader warps instead of copying them into an aligned scratch image first:
                     one launch and no scratch, for K-contiguous operands whose rows start on 8-byte boundaries. Two
                     warps of 8- and 16-byte copies deliver a small fraction of what TMA does (config 4 'nt': 279 us
                     against 43 us with the copy), so this is for callers without scratch, not for speed             */
  int32_t reserved[3];
} b200_gemm_policy;

/* One GEMM call. Replaces the argument list of the reference's jit host stub gemm_a16w16_gfx950
 * (kernels/gemm_a16w16_gfx950.py:1145-1210): out, a, b, bias, semaphore, signal, split_k, param, stream. */
typedef struct b200_gemm_args {
  const void* a;    /* device pointer to A[0,0] (storage offset already applied)                      */
  const void* b;    /* device pointer to B[0,0]; B is logically [K,N]                                 */
  void* out;        /* device pointer to C[0,0]; row-major, row stride ldo elements                   */
  const void* bias; /* device pointer to bias[N] in the input dtype, contiguous; NULL = no bias       */
  int64_t m, n, k;
  int64_t lda;       /* A leading stride in elements: row stride when a_trans == 0, column stride when 1 */
  int64_t ldb;       /* B leading stride in elements: row stride when b_trans == 0, column stride when 1 */
  int64_t ldo;       /* C row stride in elements                                                          */
  int32_t a_trans;   /* 0: 'n' A, K contiguous; 1: 't' A, M contiguous                                    */
  int32_t b_trans;   /* 0: 'n' B, N contiguous; 1: 't' B, K contiguous (stored as [N,K])                  */
  int32_t in_dtype;  /* B200_GEMM_DTYPE_BF16 or _FP16                                                      */
  int32_t out_dtype; /* in_dtype or B200_GEMM_DTYPE_FP32                                                   */
  b200_gemm_policy policy;
  void* workspace; /* device scratch of at least b200_gemm_workspace_bytes(), 256-byte aligned; its first
                      B200_GEMM_COUNTER_BYTES hold the split-K / stream-K tickets: zero them once before the first
                      call; every call that completes leaves them zero again (self-cleaning). A call that reported
                      a given-up wait through `status` may leave tickets behind: zero the region again before the
                      next call that uses this workspace                                                         */
  uint64_t workspace_bytes;
  int32_t* status; /* device int32[4], or NULL. Written only when a bounded wait inside a kernel gave up:
                      [0]=error code (1), [1]=CTA, [2]=role, [3]=unit                                         */
  uint64_t* trace; /* device uint64[trace_words], or NULL. Profiling aid: every CTA records %globaltimer stamps of its
                      producer / MMA / epilogue roles for its first 16 work items: [cta][role 0..3][item][4] (begin, first
                      data / accumulator handed back, end, and a counter: stalled waits, or clock64 for the epilogue;
                      role 3 = cycles the MMA thread spent in wait / fence / issue / commit). Needs
                      grid * 4 * 16 * 4 words; ignored when smaller; twice that many words also turns on the
                      per-K-block cycle counters (which slow the kernel down)                                            */
  uint64_t trace_words;
} b200_gemm_args;

/* What a call would do, for tests, the tuner and workspace sizing. */
typedef struct b200_gemm_plan {
  int32_t tile_m, tile_n, tile_k, stages, split_k, cta_group, swap_ab, group_m;
  int32_t tiles_p, tiles_q; /* tile grid over (128-row operand, tile_n operand)                              */
  int32_t num_units, grid;  /* work units (tile x K-slice) and persistent CTAs                               */
  int32_t smem_bytes, tmem_cols;
  int32_t cluster_split;                /* CTAs per cluster in cluster split-K mode, else 0                              */
  int32_t stream_k, sk_tiles, sk_slots; /* stream-K on; tiles cut into K spans; partial slots reserved per such tile */
  int32_t a_repacked, b_repacked; /* 1 when the operand is not TMA-encodable (base or pitch not 16-byte aligned)
                                     and is first copied into an aligned scratch image in the workspace        */
  int32_t a_loader, b_loader;     /* 1 when such an operand is instead fetched inside the GEMM kernel by its loader
                                     warps: K-contiguous rows that start on 8-byte boundaries (no copy, no scratch).
                                     The ring depth is then the variant's deepest, whatever `stages` asked for  */
  uint64_t counter_bytes, partial_bytes, repack_bytes, workspace_bytes;
  int32_t atomic_out;  /* 1: the atomic split mode is in effect (one more small launch sets C to the bias beforehand) */
  int32_t reserved;
} b200_gemm_plan;

/* Launch the GEMM on `cuda_stream` (a cudaStream_t; NULL = legacy default stream) of the current device.
 * Replaces: gemm_a16w16 -> run_cached -> gemm_a16w16_gfx950 launch
 * (kernels/gemm_a16w16_gfx950.py:1434-1440, kernels/common.py:7-39). */
int b200_gemm_a16w16(const b200_gemm_args* args, void* cuda_stream);

/* Same GEMM as b200_gemm_a16w16 for callers that are not allowed to allocate device memory: plug-ins running inside a
 * serving engine or embedded runtime that owns the whole device arena, where cudaMalloc is forbidden after start-up or
 * would fail, and that therefore cannot provide `workspace` either. It has no counterpart in the reference (whose
 * split-K scratch is a torch allocation, kernels/gemm_a16w16_gfx950.py:1277-1281).
 *   - `args->workspace` / `workspace_bytes` are ignored. The scratch a call needs (split-K / stream-K tickets and fp32
 *     partial tiles, repack images) comes from one array of B200_GEMM_STATIC_SCRATCH_BYTES built into the library; every
 *     GPU that loads the library holds that array until the process exits.
 *   - A call whose plan needs more scratch than that returns B200_GEMM_ERR_TOO_LARGE and launches nothing
 *     (b200_gemm_workspace_bytes tells the need beforehand). Calls that need no scratch are never limited. When it is
 *     the aligned copy of an operand TMA cannot describe that does not fit, the call switches policy.loader on by
 *     itself, so that such operands are fetched inside the kernel where their layout allows.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs stay the caller's.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call outside any stream capture. Later calls reuse the address.
 *   - All calls on a device share the one array, which keeps the previous call's contents; the tickets a call uses are
 *     cleared on its stream before its kernel runs. Two calls that overlap on the GPU (different streams, or different
 *     host threads without stream ordering) race on the array: serialise them. */
#define B200_GEMM_STATIC_SCRATCH_BYTES (16u << 20)
int b200_gemm_a16w16_static_scratch(const b200_gemm_args* args, void* cuda_stream);

/* Plan once, launch many times. b200_gemm_prepare does all host-side work of a call (validation, plan, tensor maps;
 * host memory only) and returns an opaque handle; b200_gemm_launch enqueues the kernels of that call on a stream of
 * the device that was current at prepare time; b200_gemm_release frees the handle. The handle stays valid while the
 * buffers named in `args` (operands, output, bias, workspace, status) stay where they are.
 * Replaces the per-policy compiled-kernel cache of run_cached (kernels/common.py:7-39) keyed on the constexpr
 * param: here the cached object is the resolved launch, not compiled code. */
typedef struct b200_gemm_handle b200_gemm_handle;
int b200_gemm_prepare(const b200_gemm_args* args, b200_gemm_handle** handle);
int b200_gemm_launch(const b200_gemm_handle* handle, void* cuda_stream);
void b200_gemm_release(b200_gemm_handle* handle);

/* Resolve the policy for these arguments without launching.
 * Replaces: make_gemm_a16w16_param_and_validate + assert_no_k_tail
 * (kernels/gemm_a16w16_gfx950.py:1213-1274). */
int b200_gemm_plan_query(const b200_gemm_args* args, b200_gemm_plan* plan);

/* Scratch bytes the call needs (0 = none). Replaces get_split_k_buffers
 * (kernels/gemm_a16w16_gfx950.py:1277-1281), whose fixed 2 x int32[256] limited split-K to 256 tiles. */
uint64_t b200_gemm_workspace_bytes(const b200_gemm_args* args);

/* Kernel variant table (for the tuner): number of compiled (tile_n, cta_group, tile_k) variants and their
 * description (tile_k = K elements per pipeline stage; the first entry of a (tile_n, cta_group) is its default).
 * Replaces the JIT cache of kernels/common.py:7-39 with an ahead-of-time table. */
int b200_gemm_num_variants(void);
int b200_gemm_describe_variant(int index, int32_t* tile_n, int32_t* cta_group, int32_t* max_stages, int32_t* tile_k);

/* out[rows, cols] = cast(in[rows, cols] (fp32) + bias[cols]); row-major contiguous, cols % 4 == 0, 16-byte aligned
 * pointers. Last step of the K-sharded multi-GPU mode (fp32 partial sums reduced over NVLink, then rounded once).
 * Restates, for that mode, the cast + bias of the reference epilogue (kernels/gemm_a16w16_gfx950.py:541-550,
 * :660-661); the reference itself has no multi-GPU path. */
int b200_gemm_cast_bias(const float* in, void* out, const void* bias, int64_t rows, int64_t cols, int32_t out_dtype,
                        int32_t bias_dtype, void* cuda_stream);

/* Fused K-sharded mode (several GPUs of one box, one process per GPU; not in the reference, which is single-GPU).
 * Rank r computes the fp32 partial product of its K slab for the rows that rank d owns and its GEMM epilogue stores
 * the tiles straight into slot r of rank d's receive buffer over NVLink: `out` of b200_gemm_a16w16 is then a pointer
 * returned by b200_peer_open. After all ranks have finished (a stream-ordered barrier of the host's choosing), the
 * owner sums its slots in index order, adds the bias and rounds once:
 * out[rows, cols] = cast(sum_s slots[s * slot_stride ...][rows, cols] + bias[cols]); slots are fp32 row-major
 * contiguous images slot_stride elements apart (slot_stride % 4 == 0), cols % 4 == 0, 16-byte aligned pointers.
 * Same rounding as the reference epilogue (kernels/gemm_a16w16_gfx950.py:541-550, :660-661). */
int b200_gemm_reduce_slots(const float* slots, int64_t slot_stride, int32_t n_slots, void* out, const void* bias,
                           int64_t rows, int64_t cols, int32_t out_dtype, int32_t bias_dtype, void* cuda_stream);

/* Peer mapping of device memory between the processes of one box (CUDA IPC). The exporting process fills a handle for
 * any pointer inside a cudaMalloc allocation (it need not be the allocation's base); the handle is plain bytes and may
 * be sent to the other processes by any host channel. b200_peer_open maps it into the calling process for the current
 * device (peer access to the exporting GPU is enabled on first use) and returns the pointer that corresponds to the
 * exported one; a process cannot open its own handle. b200_peer_close unmaps. These calls allocate no device memory and
 * launch nothing; the exporter must keep the allocation alive while any peer has it open. Kernels may store to such a pointer
 * and load from it one CTA at a time; a load that fans one fetch out to several CTAs of a cluster must never target it. */
typedef struct b200_peer_handle {
  uint8_t ipc[64];  /* cudaIpcMemHandle_t of the containing allocation */
  uint64_t offset;  /* byte offset of the exported pointer inside it   */
  uint64_t bytes;   /* bytes from the exported pointer to the end of the allocation */
  int32_t device;   /* CUDA device ordinal in the exporting process    */
  int32_t reserved;
} b200_peer_handle;
int b200_peer_export(const void* ptr, b200_peer_handle* handle);
int b200_peer_open(const b200_peer_handle* handle, void** ptr);
int b200_peer_close(void* ptr, const b200_peer_handle* handle);

/* Known-answer self-test for hosts without a test harness of their own (a plug-in loaded into another engine calls it
 * once at start-up). Runs 200 x 264 x 328 GEMMs on small-integer operands, for which fp32 accumulation is exact, through
 * every tile family (16...256 wide, CTA pairs, both stage depths, ticket and cluster split-K, stream-K, swapped operands),
 * the four layouts and both 16-bit dtypes, and compares each result bit for bit with a plain CUDA-core reference. This
 * checks exactly what a wrong tensor-map, shared-memory-descriptor or instruction-descriptor encoding would break.
 * Operands, outputs and workspace live in the library's built-in scratch array (nothing is allocated); the call
 * launches on `cuda_stream` and synchronises it. Returns B200_GEMM_OK, B200_GEMM_ERR_SELFTEST, or the error of a failing
 * launch; *failed_case (optional) receives the 1-based index of the failing case. Serialise with other users of the
 * built-in scratch. The reference has no counterpart: its descriptors are generated by FlyDSL
 * (kernels/gemm_a16w16_gfx950.py:378-705 are traced, not hand-encoded). */
int b200_gemm_selftest(void* cuda_stream, int32_t* failed_case);

/* Check of the bounded-wait mechanism every kernel of this library relies on, without running a GEMM: launches one
 * thread that waits on a shared-memory barrier nobody ever signals, with a limit of `limit_us` microseconds (1 ...
 * 1000000). The wait runs out, and the thread reports it exactly as a GEMM kernel would: status[0] = 1, status[1] = 0
 * (CTA), status[2] = 9 (role: self-test), status[3] = -1; then the kernel returns normally and the context stays
 * usable. `status` is a device int32[4] that the caller zeroed. Takes the place of the unbounded flag spin of the
 * reference's split-K protocol (kernels/gemm_a16w16_gfx950_utils.py:216-247), which has no such exit. */
int b200_gemm_wait_selftest(int32_t* status, uint32_t limit_us, void* cuda_stream);

/* Text for an error code; for B200_GEMM_ERR_LAUNCH the last CUDA error string seen by this thread. */
const char* b200_gemm_strerror(int code);

/* Library / build identification, e.g. "b200_gemm 0.1 sm_100a". */
const char* b200_gemm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_GEMM_H_ */

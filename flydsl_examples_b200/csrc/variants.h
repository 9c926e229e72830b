// The ahead-of-time table of GEMM kernel variants, spread over several translation units so that they compile side
// by side. Each accessor returns the kernel for (tile_n, stages) of its family, or null when that combination is
// not built (too much shared memory, or not on the menu).
#pragma once
#include "gemm_kernel.cuh"

namespace b200 {

constexpr int kSmemLimit = 232448;  // 227 KB opt-in dynamic shared memory per CTA on sm_100

typedef void (*KernelFn)(const GemmParams);

template <int TILE_Q, int S, int CG, int TK, bool LOADER = false>
constexpr KernelFn kfn() {
  if constexpr (SmemLayout<TILE_Q, S, CG, TK>::kDynBytes <= kSmemLimit)
    return gemm_a16w16_sm100_kernel<TILE_Q, S, CG, TK, LOADER>;
  else
    return nullptr;
}

KernelFn single_k128_variant(int tile_q, int stages);  // one CTA per tile, 128 K elements per stage: tile_n 16..128
KernelFn single_k64_variant(int tile_q, int stages);   // one CTA per tile, 64 K elements per stage: tile_n 16..256
KernelFn pair_variant(int tile_q, int stages);         // a CTA pair per 256-row tile: tile_n 128, 192, 256, 512
// Variants with cp.async loader warps, built at the deepest ring of each family only: `*stages` receives that depth.
KernelFn loader_variant(int tile_q, int cta_group, int tile_k, int* stages);

}  // namespace b200

// GEMM kernel variants with cp.async loader warps (operands whose base or pitch is a multiple of 8 but not of 16
// bytes, which TMA cannot describe). One ring depth per family: the deepest that fits.
#include "variants.h"

namespace b200 {

KernelFn loader_variant(int tile_q, int cta_group, int tile_k, int* stages) {
  struct Row {
    int tile_q, cta_group, tile_k, stages;
    KernelFn fn;
  };
  static const Row rows[] = {
      {16, 1, 128, 5, kfn<16, 5, 1, 128, true>()},   {32, 1, 128, 5, kfn<32, 5, 1, 128, true>()},
      {64, 1, 128, 4, kfn<64, 4, 1, 128, true>()},   {128, 1, 128, 3, kfn<128, 3, 1, 128, true>()},
      {16, 1, 64, 8, kfn<16, 8, 1, 64, true>()},     {32, 1, 64, 8, kfn<32, 8, 1, 64, true>()},
      {64, 1, 64, 8, kfn<64, 8, 1, 64, true>()},     {128, 1, 64, 6, kfn<128, 6, 1, 64, true>()},
      {256, 1, 64, 4, kfn<256, 4, 1, 64, true>()},   {128, 2, 64, 8, kfn<128, 8, 2, 64, true>()},
      {192, 2, 64, 6, kfn<192, 6, 2, 64, true>()},   {256, 2, 64, 6, kfn<256, 6, 2, 64, true>()},
  };
  for (const Row& r : rows) {
    if (r.tile_q == tile_q && r.cta_group == cta_group && r.tile_k == tile_k && r.fn != nullptr) {
      if (stages != nullptr) *stages = r.stages;
      return r.fn;
    }
  }
  return nullptr;
}

}  // namespace b200

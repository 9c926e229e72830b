// GEMM kernel variants: one CTA per tile, pipeline stages of 64 K elements.
#include "variants.h"

namespace b200 {

template <int TQ>
static KernelFn by_stages(int stages) {
  switch (stages) {
    case 2: return kfn<TQ, 2, 1, 64>();
    case 3: return kfn<TQ, 3, 1, 64>();
    case 4: return kfn<TQ, 4, 1, 64>();
    case 5: return kfn<TQ, 5, 1, 64>();
    case 6: return kfn<TQ, 6, 1, 64>();
    case 8: return kfn<TQ, 8, 1, 64>();
    default: return nullptr;
  }
}

KernelFn single_k64_variant(int tile_q, int stages) {
  switch (tile_q) {
    case 16: return by_stages<16>(stages);
    case 32: return by_stages<32>(stages);
    case 64: return by_stages<64>(stages);
    case 128: return by_stages<128>(stages);
    case 256: return by_stages<256>(stages);
    default: return nullptr;
  }
}

}  // namespace b200

// GEMM kernel variants: a tcgen05 cta_group::2 CTA pair per 256-row tile, pipeline stages of 64 K elements.
#include "variants.h"

namespace b200 {

template <int TQ>
static KernelFn by_stages(int stages) {
  switch (stages) {
    case 2: return kfn<TQ, 2, 2, 64>();
    case 3: return kfn<TQ, 3, 2, 64>();
    case 4: return kfn<TQ, 4, 2, 64>();
    case 5: return kfn<TQ, 5, 2, 64>();
    case 6: return kfn<TQ, 6, 2, 64>();
    case 8: return kfn<TQ, 8, 2, 64>();
    default: return nullptr;
  }
}

// 512 columns: 48 KB per stage and CTA, so four stages at most
static KernelFn wide(int stages) {
  switch (stages) {
    case 2: return kfn<512, 2, 2, 64>();
    case 3: return kfn<512, 3, 2, 64>();
    case 4: return kfn<512, 4, 2, 64>();
    default: return nullptr;
  }
}

KernelFn pair_variant(int tile_q, int stages) {
  switch (tile_q) {
    case 128: return by_stages<128>(stages);
    case 192: return by_stages<192>(stages);
    case 256: return by_stages<256>(stages);
    case 512: return wide(stages);
    default: return nullptr;
  }
}

}  // namespace b200

// The warp-level kernel for GGUF IQ2_XXS and IQ2_S (the decoder of IQ2_XS with their block layouts and grids).
#include "ffmt_iq2xs.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_iq2xxs() {
  static const FragOps ops = FragOpsOf<FragIQ2<16>>::ops();
  return &ops;
}
const FragOps *frag_ops_iq2s() {
  static const FragOps ops = FragOpsOf<FragIQ2<22>>::ops();
  return &ops;
}
}  // namespace ishi

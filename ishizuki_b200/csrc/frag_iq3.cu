// The warp-level kernel for GGUF IQ3_XXS and IQ3_S.
#include "ffmt_iq3.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_iq3xxs() {
  static const FragOps ops = FragOpsOf<FragIQ3<18>>::ops();
  return &ops;
}
const FragOps *frag_ops_iq3s() {
  static const FragOps ops = FragOpsOf<FragIQ3<21>>::ops();
  return &ops;
}
}  // namespace ishi

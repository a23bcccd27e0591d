// The warp-level kernel for four of the other GGML block types (through the dense decoder).
#include "ffmt_ggml.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_ggml_a(int type) {
  static const FragOps ops10 = FragOpsOf<FragGGML<10>>::ops();
  static const FragOps ops16 = FragOpsOf<FragGGML<16>>::ops();
  static const FragOps ops22 = FragOpsOf<FragGGML<22>>::ops();
  static const FragOps ops18 = FragOpsOf<FragGGML<18>>::ops();
  return type == 10 ? &ops10 : type == 16 ? &ops16 : type == 22 ? &ops22 : type == 18 ? &ops18 : nullptr;
}
}  // namespace ishi

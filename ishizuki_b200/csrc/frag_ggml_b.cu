// The warp-level kernel for four of the other GGML block types (through the dense decoder).
#include "ffmt_ggml.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_ggml_b(int type) {
  static const FragOps ops21 = FragOpsOf<FragGGML<21>>::ops();
  static const FragOps ops19 = FragOpsOf<FragGGML<19>>::ops();
  static const FragOps ops29 = FragOpsOf<FragGGML<29>>::ops();
  static const FragOps ops23 = FragOpsOf<FragGGML<23>>::ops();
  return type == 21 ? &ops21 : type == 19 ? &ops19 : type == 29 ? &ops29 : type == 23 ? &ops23 : nullptr;
}
}  // namespace ishi

// The warp-level kernel for GGUF Q4_K.
#include "ffmt_q4k.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_q4k() {
  static const FragOps ops = FragOpsOf<FragQ4K>::ops();
  return &ops;
}
}  // namespace ishi

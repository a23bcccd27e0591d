// The warp-level kernel for GGUF Q6_K.
#include "ffmt_q6k.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_q6k() {
  static const FragOps ops = FragOpsOf<FragQ6K>::ops();
  return &ops;
}
}  // namespace ishi

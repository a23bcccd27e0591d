// The warp-level kernel for GGUF Q2_K.
#include "ffmt_q2k.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_q2k() {
  static const FragOps ops = FragOpsOf<FragQ2K>::ops();
  return &ops;
}
}  // namespace ishi

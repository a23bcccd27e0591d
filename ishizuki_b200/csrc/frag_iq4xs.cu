// The warp-level kernel for GGUF IQ4_XS.
#include "ffmt_iq4xs.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_iq4xs() {
  static const FragOps ops = FragOpsOf<FragIQ4XS>::ops();
  return &ops;
}
}  // namespace ishi

// The warp-level kernel for GGUF IQ2_XS.
#include "ffmt_iq2xs.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_iq2xs() {
  static const FragOps ops = FragOpsOf<FragIQ2XS>::ops();
  return &ops;
}
}  // namespace ishi

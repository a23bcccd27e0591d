// The warp-level kernel for GGUF IQ1_S and IQ1_M.
#include "ffmt_iq1.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_iq1s() {
  static const FragOps ops = FragOpsOf<FragIQ1<19>>::ops();
  return &ops;
}
const FragOps *frag_ops_iq1m() {
  static const FragOps ops = FragOpsOf<FragIQ1<29>>::ops();
  return &ops;
}
}  // namespace ishi

// The tcgen05 kernel for GGUF blocks: Q4_K (the no-allocation entry point), Q6_K, IQ2_XS.
#include "ishi_row_impl.cuh"
#include "rfmt_iq2xs.cuh"
#include "rfmt_q4k.cuh"
#include "rfmt_q6k.cuh"

namespace ishi {
const RowOps *row_ops_ggml(int type) {
  static const RowOps q4k = RowOpsOf<RowQ4K>::ops(), q6k = RowOpsOf<RowQ6K>::ops(), iq2xs = RowOpsOf<RowIQ2XS>::ops();
  return type == 12 ? &q4k : type == 14 ? &q6k : type == 17 ? &iq2xs : nullptr;
}
}  // namespace ishi

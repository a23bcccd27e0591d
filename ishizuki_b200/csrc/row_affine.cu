// The tcgen05 kernel for the MLX affine packs the warp-level kernel does not take (8-bit, 2-bit
// group 32, fp32 scales).
#include "ishi_row_impl.cuh"
#include "rfmt_affine.cuh"

namespace ishi {
const RowOps *row_ops_affine(int bits) {
  static const RowOps b2 = RowOpsOf<RowAffine<2>>::ops(), b4 = RowOpsOf<RowAffine<4>>::ops(), b8 = RowOpsOf<RowAffine<8>>::ops();
  return bits == 2 ? &b2 : bits == 4 ? &b4 : bits == 8 ? &b8 : nullptr;
}
}  // namespace ishi

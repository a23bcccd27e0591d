// The warp-level kernel for MLX affine 2-bit packs (group 64 / 128, fp16 or bf16 scales), the
// ternary layout among them.
#include "ffmt_affine.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_affine2(int group_size, bool bf16) {
  static const FragOps ops[4] = {
      FragOpsOf<FragAffine<2, 64, false>>::ops(), FragOpsOf<FragAffine<2, 128, false>>::ops(),
      FragOpsOf<FragAffine<2, 64, true>>::ops(), FragOpsOf<FragAffine<2, 128, true>>::ops()};
  const int gi = group_size == 64 ? 0 : group_size == 128 ? 1 : -1;
  return gi < 0 ? nullptr : &ops[gi + (bf16 ? 2 : 0)];
}
}  // namespace ishi

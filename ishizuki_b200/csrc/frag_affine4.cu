// The warp-level kernel for MLX affine 4-bit packs (group 32 / 64 / 128, fp16 or bf16 scales).
#include "ffmt_affine.cuh"
#include "ishi_frag_impl.cuh"

namespace ishi {
const FragOps *frag_ops_affine4(int group_size, bool bf16) {
  static const FragOps ops[6] = {
      FragOpsOf<FragAffine<4, 32, false>>::ops(), FragOpsOf<FragAffine<4, 64, false>>::ops(),
      FragOpsOf<FragAffine<4, 128, false>>::ops(), FragOpsOf<FragAffine<4, 32, true>>::ops(),
      FragOpsOf<FragAffine<4, 64, true>>::ops(), FragOpsOf<FragAffine<4, 128, true>>::ops()};
  const int gi = group_size == 32 ? 0 : group_size == 64 ? 1 : group_size == 128 ? 2 : -1;
  return gi < 0 ? nullptr : &ops[gi + (bf16 ? 3 : 0)];
}
}  // namespace ishi

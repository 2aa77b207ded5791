// One slice of the tensor-core GEMM instantiations (see gemm_instances.cuh):
// the block-scaled fp8 kind, which exists for CTA pairs only: the two-accumulator
// tile of up to 192 columns and the one-accumulator tile of up to 384.
#include "gemm_instances.cuh"

namespace oxm {
cudaError_t launch_gemm_mx(const GemmLaunch &l, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC,
                           const GemmParams &p, char *name, size_t name_len) {
  if (l.bn == 256) return launch_instance<256, 6, 0, 0, 3, 1, 0>(l, tmA, tmB, tmC, p, name, name_len);
  if (l.packed) return launch_instance<512, 4, 0, 0, 3, 1, 1>(l, tmA, tmB, tmC, p, name, name_len);
  return launch_instance<512, 4, 0, 0, 3, 1, 0>(l, tmA, tmB, tmC, p, name, name_len);
}
}  // namespace oxm

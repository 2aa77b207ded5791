// One slice of the tensor-core GEMM instantiations (see gemm_instances.cuh).
#include "gemm_instances.cuh"

namespace oxm {
OXM_DEFINE_GEMM_LAUNCH(launch_gemm_f8_kn, 0, 1, 2)
}  // namespace oxm

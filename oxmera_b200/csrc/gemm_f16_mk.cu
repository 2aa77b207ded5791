// One slice of the tensor-core GEMM instantiations (see gemm_instances.cuh).
#include "gemm_instances.cuh"

namespace oxm {
OXM_DEFINE_GEMM_LAUNCH(launch_gemm_f16_mk, 1, 0, 0)
}  // namespace oxm

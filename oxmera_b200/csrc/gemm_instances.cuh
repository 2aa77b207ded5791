// Instantiation and launch of the tensor-core GEMM.  The kernel template has
// some sixty useful instantiations; they are spread over several translation
// units (one per operand type and pair of operand majors) so that they compile
// in parallel.  Each unit defines one launch function with this signature.
#pragma once

#include <cuda_runtime.h>

#include <cstdio>

#include "gemm_tcgen05.cuh"

namespace oxm {

struct GemmLaunch {
  int bn, pair;      // the instance's widest tile; CTA pairs
  bool packed;       // bn = 512: the epilogue that packs its share into registers before storing (16-bit results, whole tiles)
  bool b_mn;         // B is MN-major (both majors are fixed per translation unit; kept for the record)
  int grid;
  cudaStream_t stream;
  const CUtensorMap *sf = nullptr;  // block-scaled kind: the maps of A's and B's scale atoms
};

// Launches the instance named by `l`; writes its name into `name`.
typedef cudaError_t (*GemmLaunchFn)(const GemmLaunch &l, const CUtensorMap &tmA, const CUtensorMap &tmB,
                                    const CUtensorMap &tmC, const GemmParams &p, char *name, size_t name_len);

#define OXM_DECLARE_GEMM_LAUNCH(NAME)                                                                     \
  cudaError_t NAME(const GemmLaunch &l, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC, \
                   const GemmParams &p, char *name, size_t name_len);

OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f16_kk)   // bf16 / f16, A K-major, B K-major
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f16_kn)   // bf16 / f16, A K-major, B N-major
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f16_mk)   // bf16 / f16, A M-major, B K-major
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f16_mn)   // bf16 / f16, A M-major, B N-major
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f8_kk)    // fp8, the same four
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f8_kn)
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f8_mk)
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_f8_mn)
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_tf32)     // f32 as 3xTF32, packed K-major operands
OXM_DECLARE_GEMM_LAUNCH(launch_gemm_mx)       // block-scaled fp8 (MX), K-major operands, wide pair tile

template <int BN, int STAGES, int A_MN, int B_MN, int KIND, int PAIR, int PACKED = 0>
cudaError_t launch_instance(const GemmLaunch &l, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC,
                            const GemmParams &p, char *name, size_t name_len) {
  using L = GemmSmem<BN, STAGES, PAIR, KIND == 3>;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, A_MN, B_MN, KIND, PAIR, PACKED>;
  static_assert(L::kDynamic <= 232448, "shared memory budget of one SM");
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)l.grid, 1, 1);
  cfg.blockDim = dim3(gemm_threads(BN), 1, 1);
  cfg.dynamicSmemBytes = L::kDynamic;
  cfg.stream = l.stream;
  cudaLaunchAttribute attr[1];
  if (PAIR) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
  }
  snprintf(name, name_len, "gemm_tcgen05_%s_bn%d_s%d_%c%c_%s%s", KIND == 1 ? "tf32x3" : KIND == 2 ? "f8" : KIND == 3 ? "mxf8" : "f16",
           BN, STAGES, A_MN ? 'm' : 'k', B_MN ? 'n' : 'k', PAIR ? "pair" : "1cta", PACKED ? "_pk" : "");
  SfMaps<KIND == 3> sfm{};
  if constexpr (KIND == 3) {
    if (!l.sf) return cudaErrorInvalidValue;
    sfm.a = l.sf[0];
    sfm.b = l.sf[1];
  }
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, p, sfm);
}

// Tile shapes and their pipeline depths (every one fills 192 KiB of shared memory).
template <int A_MN, int B_MN, int KIND>
cudaError_t launch_shape(const GemmLaunch &l, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC,
                         const GemmParams &p, char *name, size_t name_len) {
  if (l.pair) {
    if (l.bn == 512) {
      if constexpr (KIND != 1) {
        if (l.packed) return launch_instance<512, 4, A_MN, B_MN, KIND, 1, 1>(l, tmA, tmB, tmC, p, name, name_len);
      }
      return launch_instance<512, 4, A_MN, B_MN, KIND, 1>(l, tmA, tmB, tmC, p, name, name_len);
    }
    if (l.bn == 256) return launch_instance<256, 6, A_MN, B_MN, KIND, 1>(l, tmA, tmB, tmC, p, name, name_len);
    return launch_instance<128, 8, A_MN, B_MN, KIND, 1>(l, tmA, tmB, tmC, p, name, name_len);
  }
  if (l.bn == 256) return launch_instance<256, 4, A_MN, B_MN, KIND, 0>(l, tmA, tmB, tmC, p, name, name_len);
  if (l.bn == 128) return launch_instance<128, 6, A_MN, B_MN, KIND, 0>(l, tmA, tmB, tmC, p, name, name_len);
  return launch_instance<64, 8, A_MN, B_MN, KIND, 0>(l, tmA, tmB, tmC, p, name, name_len);
}

#define OXM_DEFINE_GEMM_LAUNCH(NAME, A_MN, B_MN, KIND)                                                     \
  cudaError_t NAME(const GemmLaunch &l, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC, \
                   const GemmParams &p, char *name, size_t name_len) {                                     \
    return launch_shape<A_MN, B_MN, KIND>(l, tmA, tmB, tmC, p, name, name_len);                            \
  }

}  // namespace oxm

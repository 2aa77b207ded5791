// Element load/store by runtime dtype tag, and the fused epilogue every GEMM
// kernel of the backend applies to a finished dot product.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace oxm {

// dtype tags are the C ABI's: 0 f32, 6 bf16, 7 f16, 8 fp8 e4m3, 9 fp8 e5m2.
// fp8 stores round to nearest even and saturate to the largest finite value.
__device__ __forceinline__ float load_elem(const void *base, int dtype, int64_t idx) {
  if (dtype == 0) return static_cast<const float *>(base)[idx];
  if (dtype == 6) return __bfloat162float(static_cast<const __nv_bfloat16 *>(base)[idx]);
  if (dtype == 7) return __half2float(static_cast<const __half *>(base)[idx]);
  const __nv_fp8_storage_t raw = static_cast<const __nv_fp8_storage_t *>(base)[idx];
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(raw, dtype == 8 ? __NV_E4M3 : __NV_E5M2)));
}

__device__ __forceinline__ void store_elem(void *base, int dtype, int64_t idx, float v) {
  if (dtype == 0) static_cast<float *>(base)[idx] = v;
  else if (dtype == 6) static_cast<__nv_bfloat16 *>(base)[idx] = __float2bfloat16_rn(v);
  else if (dtype == 7) static_cast<__half *>(base)[idx] = __float2half_rn(v);
  else static_cast<__nv_fp8_storage_t *>(base)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, dtype == 8 ? __NV_E4M3 : __NV_E5M2);
}

// What happens to a dot product r of column `col` before it is stored:
//   r += bias[col];  r = act(r);  r += previous output   (each step optional)
// all in fp32; the sum is rounded once, to the output dtype, by the store.
struct Epilogue {
  const void *bias;     // N elements of the operand dtype, or null
  int64_t bias_stride;  // elements
  int32_t bias_dtype;
  int32_t activation;   // 0 none, 1 relu, 2 gelu (erf form)
  int32_t accumulate;   // 1: add what the output held (gradient accumulation)
  int32_t any;          // 0: nothing to do
};

__device__ __forceinline__ float apply_activation(float r, int act) {
  if (act == 1) return fmaxf(r, 0.0f);
  if (act == 2) return 0.5f * r * (1.0f + erff(r * 0.70710678118654752440f));
  return r;
}

__device__ __forceinline__ float apply_epilogue(const Epilogue &e, float r, int64_t col, const void *out, int out_dtype,
                                                int64_t out_idx) {
  if (e.bias) r += load_elem(e.bias, e.bias_dtype, col * e.bias_stride);
  r = apply_activation(r, e.activation);
  if (e.accumulate) r += load_elem(out, out_dtype, out_idx);
  return r;
}

}  // namespace oxm

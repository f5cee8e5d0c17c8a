// Loads / stores through a runtime dtype code (VILA_DT_BF16 = 0, VILA_DT_F32 = 1) and the exact
// (non-approximate) fp32 gate functions used where a model asks for 32-bit arithmetic.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace vb {

__device__ __forceinline__ float ld_any(const void* p, int dt, size_t i) {
  return dt ? static_cast<const float*>(p)[i]
            : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_any(void* p, int dt, size_t i, float v) {
  if (dt) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
// A load that leaves the element's bits untouched: nothing consumes the result, so a thread can have many of
// them in flight (ld_any converts at once and waits for each load in turn); raw_to_float converts later.
__device__ __forceinline__ uint32_t ld_raw(const void* p, int dt, size_t i) {
  return dt ? __float_as_uint(static_cast<const float*>(p)[i])
            : static_cast<uint32_t>(static_cast<const unsigned short*>(p)[i]);
}
__device__ __forceinline__ float raw_to_float(uint32_t raw, int dt) {
  return __uint_as_float(dt ? raw : raw << 16);
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_exact_f(float z) { return z / (1.0f + expf(-z)); }

}  // namespace vb

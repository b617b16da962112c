// Device helpers shared by the forward and backward attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace acct {

constexpr float kNegInf = -INFINITY;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

template <bool BF16>
__device__ __forceinline__ float load16(const void* base, int64_t idx) {
  if constexpr (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  else return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__device__ __forceinline__ float load_mask_value(const void* base, int dtype, int64_t idx) {
  if (dtype == 2 /*U8*/) return static_cast<float>(reinterpret_cast<const uint8_t*>(base)[idx]);
  if (dtype == 1 /*BF16*/) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

}  // namespace acct

// Shared device helpers for the Universal Attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ua {

// Constants of the operator (universal_attention_autograd.py:26-28, :85).
__device__ __forceinline__ float mask_value() { return -1e12f; }
__device__ __forceinline__ float clamp_hi() { return 0.999999f; }   // fp32 rounding of 1 - 1e-6
__device__ __forceinline__ float clamp_lo_bwd() { return 1e-6f; }

struct Shape {
  int B, H, R, N, C, D, L;
};

template <typename T> struct Num;
template <> struct Num<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float rnd(float v) { return v; }
};
template <> struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

}  // namespace ua

// Element-type helpers for kernels that are instantiated for bf16 and for fp32 activations / weights
// (the serving path runs a model either in bf16 with fp32 accumulation or entirely in fp32).
#pragma once
#include "util.cuh"

namespace llmctl {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

}  // namespace llmctl

// Dispatch a templated launch on the `is_fp32` flag of the C ABI.
#define LLMCTL_DISPATCH_DTYPE(is_fp32, T, ...) \
  do {                                         \
    if (is_fp32) {                             \
      using T = float;                         \
      __VA_ARGS__;                             \
    } else {                                   \
      using T = __nv_bfloat16;                 \
      __VA_ARGS__;                             \
    }                                          \
  } while (0)

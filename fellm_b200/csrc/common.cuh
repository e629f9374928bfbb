// Shared device helpers for the fellm_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FELLM_API extern "C" __attribute__((visibility("default")))

// Launchers return 0 on success, a positive cudaError_t, or one of these negative codes.
#define FELLM_ERR_SIZE (-1)      // a size the kernel does not take
#define FELLM_ERR_ARG (-2)       // a null or inconsistent argument

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return (int)e;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

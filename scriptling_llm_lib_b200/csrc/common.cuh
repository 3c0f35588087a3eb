// Shared device helpers for the sm_100a kernels: element conversion, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SLLM_PAGE 64  // tokens per cache page; the Python side asserts the same number

#define SLLM_EXPORT extern "C" __attribute__((visibility("default")))

// Every launcher returns the CUDA error code of its launch (0 = success); negative values are
// argument errors detected on the host before anything is enqueued.
#define SLLM_ERR_ARG (-1)
#define SLLM_RETURN_LAST() return (int)cudaGetLastError()

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// weights of a norm may be stored in bfloat16 or float32 whatever the activation type
__device__ __forceinline__ float load_w(const void* w, int is_f32, int j) {
  return is_f32 ? ((const float*)w)[j] : __bfloat162float(((const bf16*)w)[j]);
}

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

// Sum over the block, same value returned to every thread; fixed order, so a row's result does
// not depend on what else is in the batch. `red` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// A measuring stick for the 32-bit path: the rate at which this GPU does dependent-free float
// fused multiply-adds, which no file of measured peaks provides. Every thread runs eight
// independent chains; nothing touches memory until the end. The reference has nothing like it
// (it runs on CPUs); bench.py divides the 32-bit prompt step's rate by this one.
#include "common.cuh"

__global__ void __launch_bounds__(256) fma_loop_kernel(float* __restrict__ out, int iters, float b, float c) {
  float a[8];
#pragma unroll
  for (int j = 0; j < 8; j++) a[j] = (float)(threadIdx.x + j) * 1e-3f;
  for (int i = 0; i < iters; i++) {
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = fmaf(a[j], b, c);
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; j++) s += a[j];
  out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = s;
}

// `out` holds blocks * 256 floats; the launch does blocks * 256 * iters * 16 floating-point operations.
SLLM_EXPORT int sllm_fma_loop(float* out, int blocks, int iters, cudaStream_t stream) {
  if (blocks <= 0 || iters <= 0) return SLLM_ERR_ARG;
  fma_loop_kernel<<<blocks, 256, 0, stream>>>(out, iters, 0.999f, 1e-4f);
  SLLM_RETURN_LAST();
}

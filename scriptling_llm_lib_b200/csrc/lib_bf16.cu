// The generic kernel set on bfloat16 elements (float accumulation): the shapes the fast
// bfloat16 kernels do not take, and the conversions between the two element types.
#include "generic_kernels.cuh"
#define ELEM bf16
#define FN(name) sllm_##name##_bf16
#include "generic_launchers.inc"

SLLM_EXPORT int sllm_cast_bf16_to_f32(const void* in, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_kernel<bf16, float><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const bf16*)in, (float*)out, (size_t)n);
  SLLM_RETURN_LAST();
}
SLLM_EXPORT int sllm_cast_f32_to_bf16(const void* in, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_kernel<float, bf16><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const float*)in, (bf16*)out, (size_t)n);
  SLLM_RETURN_LAST();
}

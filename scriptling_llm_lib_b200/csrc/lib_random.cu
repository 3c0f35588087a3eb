// Random-weights mode on the device: fills a tensor from a seed without the values ever crossing
// the bus. The reference has no such mode (its only weight source is a GGUF file,
// model_f32.go:133-293). Element e of tensor number `index` is drawn from Philox4x32-10 with key
// (low word of the seed, index) and counter (e / 4 as two words, high word of the seed, 0): word
// pair (0,1) of the output gives elements 4c and 4c+1 as the cosine and sine branch of a Box-Muller
// pair, word pair (2,3) gives 4c+2 and 4c+3. value = mean + std * z in double, rounded once to
// float and, for bfloat16 storage, once more. weights/random_init.py states the same on the host.
#include "common.cuh"
#include "philox.cuh"

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, unsigned seed_lo, unsigned seed_hi, unsigned index,
                                   double mean, double std) {
  long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long e0 = c * 4;
  if (e0 >= n) return;
  Philox4 r = philox4x32_10((unsigned)c, (unsigned)(c >> 32), seed_hi, 0u, seed_lo, index);
  double z[4];
  exact_normal_pair(r.w[0], r.w[1], &z[0], &z[1]);
  exact_normal_pair(r.w[2], r.w[3], &z[2], &z[3]);
#pragma unroll
  for (int j = 0; j < 4; j++)
    if (e0 + j < n) out[e0 + j] = from_f32<T>(__double2float_rn(__dadd_rn(mean, __dmul_rn(std, z[j]))));
}

__global__ void fill_integer_kernel(int* __restrict__ out, long long n, unsigned seed_lo, unsigned seed_hi, unsigned index,
                                    unsigned modulus) {
  long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long e0 = c * 4;
  if (e0 >= n) return;
  Philox4 r = philox4x32_10((unsigned)c, (unsigned)(c >> 32), seed_hi, 0u, seed_lo, index);
#pragma unroll
  for (int j = 0; j < 4; j++)
    if (e0 + j < n) out[e0 + j] = (int)(r.w[j] % modulus);
}

// kind: 0 float32, 1 bfloat16
SLLM_EXPORT int sllm_fill_normal(void* out, int kind, long long n, unsigned long long seed, unsigned index, double mean,
                                 double std, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (kind != 0 && kind != 1) return SLLM_ERR_ARG;
  long long counters = (n + 3) / 4;
  unsigned blocks = (unsigned)((counters + 255) / 256);
  unsigned lo = (unsigned)seed, hi = (unsigned)(seed >> 32);
  if (kind == 0) fill_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, lo, hi, index, mean, std);
  else fill_normal_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)out, n, lo, hi, index, mean, std);
  SLLM_RETURN_LAST();
}

SLLM_EXPORT int sllm_fill_integer(int* out, long long n, unsigned long long seed, unsigned index, unsigned modulus,
                                  cudaStream_t stream) {
  if (n <= 0) return 0;
  if (modulus == 0) return SLLM_ERR_ARG;
  long long counters = (n + 3) / 4;
  fill_integer_kernel<<<(unsigned)((counters + 255) / 256), 256, 0, stream>>>(out, n, (unsigned)seed, (unsigned)(seed >> 32),
                                                                               index, modulus);
  SLLM_RETURN_LAST();
}

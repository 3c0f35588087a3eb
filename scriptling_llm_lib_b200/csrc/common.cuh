// Shared device helpers for the sm_100a kernels: element conversion, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define SLLM_PAGE 64  // tokens per cache page; the Python side asserts the same number

#define SLLM_EXPORT extern "C" __attribute__((visibility("default")))

// every library says which page size it was built with; the loader compares it with the cache's
SLLM_EXPORT int sllm_page_tokens(void) { return SLLM_PAGE; }

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

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched through sllm_launch may be scheduled while the kernel before it in the stream
// is still draining: its blocks start, do whatever does not depend on earlier kernels (fetch
// weights), and call pdl_wait() before they touch anything an earlier kernel wrote. Every kernel
// launched this way calls pdl_launch_dependents() first and pdl_wait() before its first dependent
// access, so completion stays transitive along the stream. Launched the ordinary way, both are no-ops.
// The first kernel of a model step (the embedding) is launched the ordinary way: what earlier steps wrote
// (the cached keys and values) is complete and visible to every kernel of the step, also before its wait.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Loads of data that an earlier kernel of the stream wrote. Under programmatic dependent launch
// this kernel's lifetime overlaps the writer's, so the read-only (non-coherent, `ld.global.nc` /
// __ldg) path must not be used for them, and the compiler must not move them above pdl_wait():
// ordinary coherent loads, as volatile asm with a memory clobber. `ld_dep16_stream` does not
// allocate in L1 (data read once).
__device__ __forceinline__ uint4 ld_dep16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_dep16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_dep(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bf16 ld_dep(const bf16* p) {
  unsigned short v;
  asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return __ushort_as_bfloat16(v);
}

// four / eight consecutive elements as floats
__device__ __forceinline__ float4 ld_dep4(const float* p) {
  float4 v;
  asm volatile("ld.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_dep4(const bf16* p) {
  uint32_t a, b;
  asm volatile("ld.global.v2.u32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "l"(p) : "memory");
  __nv_bfloat162 lo = *(__nv_bfloat162*)&a, hi = *(__nv_bfloat162*)&b;
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  uint2 r = *(const uint2*)p;
  __nv_bfloat162 lo = *(__nv_bfloat162*)&r.x, hi = *(__nv_bfloat162*)&r.y;
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
// the same for data that is read once (weights streaming through): not kept in L1, so that what is
// read again and again beside it (the step's few activation rows) stays there
__device__ __forceinline__ float4 ld4_stream(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld4_stream(const bf16* p) {
  uint32_t a, b;
  asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "l"(p));
  __nv_bfloat162 lo = *(__nv_bfloat162*)&a, hi = *(__nv_bfloat162*)&b;
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *(uint32_t*)&lo;
  r.y = *(uint32_t*)&hi;
  *(uint2*)p = r;
}
struct F8 { float f[8]; };
__device__ __forceinline__ F8 ld8(const float* p) {
  F8 r;
  float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  r.f[0] = a.x; r.f[1] = a.y; r.f[2] = a.z; r.f[3] = a.w; r.f[4] = b.x; r.f[5] = b.y; r.f[6] = b.z; r.f[7] = b.w;
  return r;
}
__device__ __forceinline__ F8 ld8(const bf16* p) {
  F8 r;
  uint4 v = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int i = 0; i < 4; i++) { r.f[2 * i] = __low2float(h[i]); r.f[2 * i + 1] = __high2float(h[i]); }
  return r;
}
__device__ __forceinline__ void st8(float* p, const F8& r) {
  *(float4*)p = make_float4(r.f[0], r.f[1], r.f[2], r.f[3]);
  *(float4*)(p + 4) = make_float4(r.f[4], r.f[5], r.f[6], r.f[7]);
}
__device__ __forceinline__ void st8(bf16* p, const F8& r) {
  uint4 v;
  __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(r.f[2 * i], r.f[2 * i + 1]);
  *(uint4*)p = v;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t sllm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  static const bool off = getenv("SLLM_NO_PDL") != nullptr;   // launch the ordinary, fully serialised way
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = off ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

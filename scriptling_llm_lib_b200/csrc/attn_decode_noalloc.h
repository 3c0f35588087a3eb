/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (which has no GPU code and no notion of
 * scratch memory); it exists for users of this library.
 *
 * Who needs it: code that must not enter the CUDA allocator while it runs -- a callback of another
 * library, a loop with a latency bound that cudaMalloc's implicit synchronisation would break, or
 * a program that has given all device memory to an arena of its own and has none left to hand to
 * cudaMalloc. The ordinary entry point, sllm_attn_decode_bf16, asks its caller for scratch for the
 * per-split partial results; this one keeps that scratch in a fixed array inside the library.
 *
 *   int sllm_attn_decode_bf16_noalloc(q, q_ld, out, seq_pos0, block_table, max_pages, kpages, vpages,
 *                                     B, H, G, hd, window, scale, n_split, stream);
 *
 * Inputs and outputs are the caller's, exactly as for sllm_attn_decode_bf16 (bfloat16 queries
 * [B, q_ld], output [B, H*hd], int32 positions and block table, paged keys and values); only the
 * scratch argument is gone. It returns 0 on success, a positive cudaError_t, or a negative code
 * that sllm_attn_decode_noalloc_strerror() turns into words.
 *
 * Limits and rules:
 *  - The array holds SLLM_NOALLOC_SCRATCH_FLOATS floats (4 MiB). Every GPU on which the library is
 *    loaded holds that much until the process exits. A call needs B * H * n_split * (hd + 2)
 *    floats; more than the array holds is refused with SLLM_NOALLOC_ERR_TOO_LARGE and nothing runs.
 *  - The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
 *    that device current) and remembers it. Make that first call before any stream capture.
 *  - It calls no cudaMalloc, cudaFree or any routine that allocates.
 *  - All calls share the one array, and it keeps what the last call wrote. Nothing in it has to be
 *    zero beforehand (each call overwrites every entry it later reads), but two calls that overlap
 *    on the GPU -- different streams, or concurrent host threads -- race on it: serialise them.
 */
#ifndef SLLM_ATTN_DECODE_NOALLOC_H
#define SLLM_ATTN_DECODE_NOALLOC_H

#include <cuda_runtime.h>

#define SLLM_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define SLLM_NOALLOC_ERR_TOO_LARGE (-10)
#define SLLM_NOALLOC_ERR_DEVICE (-11)

#ifdef __cplusplus
extern "C" {
#endif

int sllm_attn_decode_bf16_noalloc(const void* q, int q_ld, void* out, const int* seq_pos0, const int* block_table,
                                  int max_pages, const void* kpages, const void* vpages, int B, int H, int G, int hd,
                                  int window, float scale, int n_split, cudaStream_t stream);
const char* sllm_attn_decode_noalloc_strerror(int code);
long long sllm_attn_decode_noalloc_capacity_floats(void);

#ifdef __cplusplus
}
#endif
#endif

// bfloat16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T, float accumulation.
// Three kernels, one set of epilogues:
//   gemm_tc_pair_kernel    more than 128 rows and columns: two SMs (a cluster of two blocks,
//                          cta_group::2) on one 256 x 256 tile;
//   gemm_tc_kernel         the one-SM form, 128 x BN tiles: narrow outputs, and wide ones of few rows;
//   gemm_tc_skinny_kernel  at most 128 rows: the weights are the 128-row operand.
//
// The one-SM kernel, which the others vary: one block per SM walks over 128 x BN output tiles. Warp
// 0 feeds shared memory with TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast), warp 1
// issues tcgen05.mma from one thread with the accumulator in tensor memory, warps 2-5 read the
// accumulator back with tcgen05.ld and write the result (as bfloat16, as float, through the SiLU
// gate when gate and up columns alternate in groups of 8, or as rotated queries and cache rows). Two
// accumulators take turns, so one tile's epilogue overlaps the next tile's products. Hand-over is
// by mbarriers: TMA completes `full[s]`, the MMA's commit arrives on `empty[s]`, a tile's last
// commit on `acc_full[a]`, the epilogue warps on `acc_empty[a]`. Rows and columns past M, N, K are
// zero-filled by TMA and masked at the store, so every size with K % 8 == 0 is taken.
//
// Replaces the reference's dense matmul (float32_ops.go:462-482) for the prompt step's
// projections (model_f32.go:391-396, :469-470, :479-493, :519-524).
//
// Every wait has a time limit; when one runs out the kernel raises *err, waits (again bounded) for
// its own copies in flight, frees its tensor memory and returns.
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

#define TC_EPI_STORE 0
#define TC_EPI_SWIGLU 1
#define TC_EPI_RESID 2      // C is the float residual stream: it receives the product; TcFold says what else is written
#define TC_EPI_QKV_ROPE 3   // C's columns are [q heads | k heads | v heads]: rotate q and k, put k and v into the cache

// The two halves of an RMSNorm folded into the products around it (a row's 1/rms is one number, so
// (v / rms * w) W^T = (1 / rms) * ((v * w) W^T); float32_ops.go:159-172 with the scale moved behind the
// sum over k). All pointers null: nothing folded.
struct TcFold {
  // in: the rows of A are v * w of a norm whose scale is still owed: sumsq_in[n_in][M] are partial sums of v^2
  // over its `1 / inv_width` columns; the accumulator's rows are multiplied by rsqrt(sum * inv_width + eps)
  const float* sumsq_in;
  int n_in;
  float inv_width, eps;
  // out (TC_EPI_RESID): C[M][ldc] += product; xb[M][N] = bfloat16(C * norm_w); sumsq_out[ceil(N/128)][M] = the
  // sums of C^2 over each 128 columns
  const float* norm_w;
  bf16* xb;
  float* sumsq_out;
};

// the scale a row is owed by a folded norm before the product: its partial sums added in their order
__device__ __forceinline__ float tc_row_scale(const TcFold& fd, int row, int M) {
  if (fd.sumsq_in == nullptr || row >= M) return 1.f;
  float sq = 0.f;
  for (int pt = 0; pt < fd.n_in; pt++) sq += fd.sumsq_in[(size_t)pt * M + row];
  return rsqrtf(sq * fd.inv_width + fd.eps);
}
__device__ __forceinline__ void tc_scale32(uint32_t (&r)[32], float rs) {
#pragma unroll
  for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) * rs);
}

// What the q|k|v epilogue needs besides the product: where each row (token) sits, the rotary
// table, the paged cache of the layer. Queries are rotated and written to C; keys are rotated and
// written, with the values, at the token's place in the cache (and not to C): the work of the
// rotary kernel (float32_ops.go:174-188, model_f32.go:445-448) without reading q|k|v again.
struct TcRope {
  const int* tok_pos;       // [M] position of each row in its sequence
  const int* tok_seq;       // [M] which row of the block table
  const int* block_table;   // [sequences][max_pages]
  int max_pages;
  const float2* cs;         // [positions][rot/2] (cos, sin)
  bf16* kpages;             // [pages][G][PAGE][hd]
  bf16* vpages;
  int H, G, hd, rot, interleaved;
};

__device__ __forceinline__ float bf16_round(uint32_t f32_bits) {
  return __bfloat162float(__float2bfloat16_rn(__uint_as_float(f32_bits)));
}

// 32 consecutive columns of one row, already final: to C (a query head), or to the row's place in
// the key or value pages.
__device__ __forceinline__ void qkv_store32(const TcRope& rp, void* C, int ldc, int row, int col, size_t cache_row,
                                            const float (&v)[32]) {
  int hidx = col / rp.hd, d0 = col % rp.hd;
  bf16* dst;
  if (hidx < rp.H) dst = (bf16*)C + (size_t)row * ldc + col;
  else if (hidx < rp.H + rp.G) dst = rp.kpages + (cache_row + (size_t)(hidx - rp.H) * SLLM_PAGE) * rp.hd + d0;
  else dst = rp.vpages + (cache_row + (size_t)(hidx - rp.H - rp.G) * SLLM_PAGE) * rp.hd + d0;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
    o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1; o.z = *(uint32_t*)&p2; o.w = *(uint32_t*)&p3;
    *(uint4*)(dst + j) = o;
  }
}

// Writes 32 consecutive accumulator columns of one row. EPI_STORE: as they are; EPI_SWIGLU: the 32
// columns are 8 gate, 8 up, 8 gate, 8 up, and 16 gated values go to column (col / 2).
template <int EPI>
__device__ __forceinline__ void tc_store_row(void* C, int row, int col, int N, int ldc, int out_f32, const uint32_t (&r)[32]) {
  if (EPI == TC_EPI_STORE) {
    if (out_f32) {
      float* dst = (float*)C + (size_t)row * ldc + col;
      if (col + 32 <= N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *(float4*)(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) if (col + j < N) dst[j] = __uint_as_float(r[j]);
      }
    } else {
      bf16* dst = (bf16*)C + (size_t)row * ldc + col;
      if (col + 32 <= N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 v;
          __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
          __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
          __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
          v.x = *(uint32_t*)&p0; v.y = *(uint32_t*)&p1; v.z = *(uint32_t*)&p2; v.w = *(uint32_t*)&p3;
          *(uint4*)(dst + j) = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) if (col + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
    }
  } else {
    int ocol = col >> 1, n_out = N >> 1;
    bf16* dst = (bf16*)C + (size_t)row * ldc + ocol;
    float h[16];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float g = __uint_as_float(r[16 * t + j]), u = __uint_as_float(r[16 * t + 8 + j]);
        h[8 * t + j] = __fdividef(g, 1.0f + __expf(-g)) * u;
      }
    if (ocol + 16 <= n_out && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 16; j += 8) {
        uint4 v;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(h[j], h[j + 1]), p1 = __floats2bfloat162_rn(h[j + 2], h[j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(h[j + 4], h[j + 5]), p3 = __floats2bfloat162_rn(h[j + 6], h[j + 7]);
        v.x = *(uint32_t*)&p0; v.y = *(uint32_t*)&p1; v.z = *(uint32_t*)&p2; v.w = *(uint32_t*)&p3;
        *(uint4*)(dst + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; j++) if (ocol + j < n_out) dst[j] = __float2bfloat16_rn(h[j]);
    }
  }
}

// One warp's share of a finished 128-row accumulator (tensor-memory columns from `acc`, lanes
// 32 q .. 32 q + 31 = rows m0 + 32 q .., columns c_lo .. c_hi - 1 = output columns n0 + c_lo ..):
// read back with tcgen05.ld and written as EPI says. c_lo and c_hi are multiples of 32, and of the
// head width in the q|k|v epilogue.
template <int EPI>
__device__ __forceinline__ void tc_epilogue_tile(uint32_t acc, int q, int lane, int m0, int n0, int c_lo, int c_hi,
                                                 void* __restrict__ C, int M, int N, int ldc, int out_f32, const TcRope& rp,
                                                 const TcFold& fd) {
  int row = m0 + q * 32 + lane;
  const bool owed = fd.sumsq_in != nullptr;
  const float rs = tc_row_scale(fd, row, M);
  if constexpr (EPI == TC_EPI_QKV_ROPE) {
    const uint32_t trow = acc + ((uint32_t)(q * 32) << 16);
    int pos = 0;
    size_t cache_row = 0;                  // (page * G) * PAGE + place in the page; + g * PAGE, times hd, is the row's place
    if (row < M) {
      pos = rp.tok_pos[row];
      int page = rp.block_table[(size_t)rp.tok_seq[row] * rp.max_pages + pos / SLLM_PAGE];
      cache_row = (size_t)page * rp.G * SLLM_PAGE + (pos % SLLM_PAGE);
    }
    const float2* csr = rp.cs + (size_t)pos * (rp.rot >> 1);
    if (rp.interleaved) {
      // pairs of adjacent columns: a chunk of 32 columns holds 16 whole pairs
#pragma unroll 1
      for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        if (n0 + c0 >= N) break;
        uint32_t r[32];
        tmem_ld32(trow + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (owed) tc_scale32(r, rs);
        if (row < M) {
          int col = n0 + c0, d0 = col % rp.hd;
          bool rotate = col / rp.hd < rp.H + rp.G;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float x0 = bf16_round(r[j]), x1 = bf16_round(r[j + 1]);
            if (rotate && d0 + j < rp.rot) {
              float2 cs = csr[(d0 + j) >> 1];
              v[j] = x0 * cs.x - x1 * cs.y;
              v[j + 1] = x0 * cs.y + x1 * cs.x;
            } else {
              v[j] = x0;
              v[j + 1] = x1;
            }
          }
          qkv_store32(rp, C, ldc, row, col, cache_row, v);
        }
        __syncwarp();
      }
    } else {
      // pairs (i, i + hd/2), the whole head rotated: two chunks of 32 columns half a head apart
      const int half = rp.hd >> 1;
#pragma unroll 1
      for (int h0 = c_lo; h0 < c_hi; h0 += rp.hd) {
        if (n0 + h0 >= N) break;
#pragma unroll 1
        for (int i0 = 0; i0 < half; i0 += 32) {
          uint32_t r0[32], r1[32];
          tmem_ld32(trow + (uint32_t)(h0 + i0), r0);
          tmem_ld32(trow + (uint32_t)(h0 + half + i0), r1);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (owed) { tc_scale32(r0, rs); tc_scale32(r1, rs); }
          if (row < M) {
            int col = n0 + h0 + i0;
            bool rotate = col / rp.hd < rp.H + rp.G;
            float v0[32], v1[32];
            const float4* c4 = (const float4*)(csr + i0);     // (cos, sin) of two pairs per load
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float4 cs = rotate ? c4[j >> 1] : make_float4(1.f, 0.f, 1.f, 0.f);
              float a0 = bf16_round(r0[j]), b0 = bf16_round(r1[j]), a1 = bf16_round(r0[j + 1]), b1 = bf16_round(r1[j + 1]);
              v0[j] = a0 * cs.x - b0 * cs.y;
              v1[j] = a0 * cs.y + b0 * cs.x;
              v0[j + 1] = a1 * cs.z - b1 * cs.w;
              v1[j + 1] = a1 * cs.w + b1 * cs.z;
            }
            qkv_store32(rp, C, ldc, row, col, cache_row, v0);
            qkv_store32(rp, C, ldc, row, col + half, cache_row, v1);
          }
          __syncwarp();
        }
      }
    }
  } else {
#pragma unroll 1
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
      if (n0 + c0 >= N) break;               // uniform over the warp
      uint32_t r[32];
      tmem_ld32(acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (owed) tc_scale32(r, rs);
      if (row < M) tc_store_row<EPI>(C, row, n0 + c0, N, ldc, out_f32, r);
    }
  }
}

// TC_EPI_RESID for one warp's share of an accumulator (rows m0 + 32 q .., columns c_lo .. c_hi - 1, both
// multiples of 128; N a multiple of 32): C += product, xb = bfloat16(C * norm_w), and the sums of C^2 of each
// span of 128 columns. An accumulator row lives in one thread, but the float residual stream wants whole
// rows of 128 bytes at a time: each chunk of 32 x 32 values goes through `stage` (4 KB of shared memory of
// this warp, 16-byte groups swizzled by the row) and comes back with eight lanes to a row.
// The first chunk's residual values are asked for before the wait for the accumulator (`acc_bar`, `parity`):
// false if that wait gave up.
__device__ __forceinline__ bool tc_epilogue_resid(uint32_t acc, int q, int lane, int m0, int n0, int c_lo, int c_hi,
                                                  float* __restrict__ C, int M, int N, int ldc, const TcFold& fd, float* stage,
                                                  uint32_t acc_bar, uint32_t parity, volatile int* abort) {
  const int row_own = m0 + q * 32 + lane;
  const float rs = tc_row_scale(fd, row_own, M);
  const bool owed = fd.sumsq_in != nullptr;
  const int sub = lane >> 3, gq = lane & 7;            // on the way back: row 4 it + sub of the chunk, columns 4 gq .. 4 gq + 3
  float sq[8];
#pragma unroll
  for (int it = 0; it < 8; it++) sq[it] = 0.f;
  // the residual values of a chunk are asked for a chunk ahead, all eight rows' at once: their way from L2
  // is what this epilogue would otherwise spend its time on
  auto load_res = [&](float4 (&v)[8], int c0) {
#pragma unroll
    for (int it = 0; it < 8; it++) {
      const int row = m0 + q * 32 + 4 * it + sub;
      v[it] = (row < M && n0 + c0 < N) ? *(const float4*)(C + (size_t)row * ldc + n0 + c0 + 4 * gq) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  float4 cur[8], nxt[8];
  load_res(cur, c_lo);
  if (!mbar_wait(acc_bar, parity, abort)) return false;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
  for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
    if (c0 + 32 < c_hi) load_res(nxt, c0 + 32);
    if (n0 + c0 < N) {                                   // uniform over the warp
      uint32_t r[32];
      tmem_ld32(acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (owed) tc_scale32(r, rs);
#pragma unroll
      for (int k = 0; k < 8; k++)
        *(float4*)(stage + lane * 32 + ((k ^ (lane & 7)) << 2)) =
            make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]), __uint_as_float(r[4 * k + 2]), __uint_as_float(r[4 * k + 3]));
      __syncwarp();
      const int col = n0 + c0 + 4 * gq;
      const float4 w = *(const float4*)(fd.norm_w + col);
#pragma unroll
      for (int it = 0; it < 8; it++) {
        const int rr = 4 * it + sub, row = m0 + q * 32 + rr;
        const float4 y = *(const float4*)(stage + rr * 32 + ((gq ^ (rr & 7)) << 2));
        if (row < M) {
          float4 v = cur[it];
          v.x += y.x; v.y += y.y; v.z += y.z; v.w += y.w;
          *(float4*)(C + (size_t)row * ldc + col) = v;
          sq[it] += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
          __nv_bfloat162 p0 = __floats2bfloat162_rn(v.x * w.x, v.y * w.y), p1 = __floats2bfloat162_rn(v.z * w.z, v.w * w.w);
          *(uint2*)(fd.xb + (size_t)row * N + col) = make_uint2(*(uint32_t*)&p0, *(uint32_t*)&p1);
        }
      }
      __syncwarp();
    }
#pragma unroll
    for (int it = 0; it < 8; it++) cur[it] = nxt[it];
    if (((c0 + 32) & 127) == 0) {                        // the end of a span of 128 columns: eight lanes hold a row's sum
      const int span = (n0 + c0) >> 7;
#pragma unroll
      for (int it = 0; it < 8; it++) {
        float t = sq[it];
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 4);
        const int row = m0 + q * 32 + 4 * it + sub;
        if (gq == 0 && row < M && span < ((N + 127) >> 7)) fd.sumsq_out[(size_t)span * M + row] = t;
        sq[it] = 0.f;
      }
    }
  }
  return true;
}

// Persistent: each block walks over output tiles (tile = blockIdx.x, += gridDim.x; consecutive
// tiles share a weight tile so it is read from HBM once and found in L2 by the others). The
// shared-memory ring runs on across tiles, and two accumulators in tensor memory take turns, so
// the epilogue of one tile overlaps the products of the next.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ C,
               int M, int N, int K, int ldc, int out_f32, int* __restrict__ err, const TcRope rp, const TcFold fd) {
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  volatile int* abort = (volatile int*)(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES, acc_empty0 = acc_full0 + 16;

  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + BN - 1) / BN, n_tiles = tiles_m * tiles_n;
  const int nkb = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 4); }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                       // k-blocks issued so far, over all tiles of this block
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < nkb; kb++, it++) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, abort);
          if (!ok) break;
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          uint32_t a_dst = smem_base + s * STAGE_BYTES;
          tma_load_2d(a_dst, &map_a, kb * TC_BK, m0, full0 + 8 * s);
          tma_load_2d(a_dst + A_BYTES, &map_b, kb * TC_BK, n0, full0 + 8 * s);
        }
      }
      if (*abort) {
        // copies already issued still land in this block's shared memory: wait for them (bounded)
        volatile int never = 0;
        for (int j = max(0, it - STAGES); j < it; j++) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1, &never);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
      int it = 0, i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, i++) {
        int a = i & 1;
        ok = mbar_wait(acc_empty0 + 8 * a, ((i >> 1) & 1) ^ 1, abort);     // the epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t acc = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < nkb; kb++, it++) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint32_t a_addr = smem_base + s * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++)
            umma_bf16(acc, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc, (kb | k) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);
        }
        if (ok) umma_commit(acc_full0 + 8 * a);
      }
    }
  } else {
    int q = warp & 3;                          // the quarter of tensor memory this warp may read
    int i = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
      int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
      int a = i & 1;
      if (!mbar_wait(acc_full0 + 8 * a, (i >> 1) & 1, abort)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      tc_epilogue_tile<EPI>(tmem_base + (uint32_t)(a * BN), q, lane, m0, n0, 0, BN, C, M, N, ldc, out_f32, rp, fd);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * a) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort) atomicExch(err, 2);
}

// ------------------------------------------------------------------ host side
template <int BN, int STAGES, int EPI>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int ldc, int out_f32,
                     int* err, cudaStream_t stream, const TcRope& rp = TcRope{}, const TcFold& fd = TcFold{}) {
  constexpr size_t smem = STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024 + 256;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 1;
  }
  int n_tiles = ((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
  dim3 grid(n_tiles < sms ? n_tiles : sms);
  gemm_tc_kernel<BN, STAGES, EPI><<<grid, TC_THREADS, smem, stream>>>(ma, mb, C, M, N, K, ldc, out_f32, err, rp, fd);
  SLLM_RETURN_LAST();
}

// ------------------------------------------------------------------ two SMs on one tile
// The two-SM form of the kernel above (tcgen05 cta_group::2): the two blocks of a cluster share a
// 256 x 256 tile. Each block loads its own 128 rows of A and its own 128 of the tile's 256 rows of
// B, the block of rank 0 issues the products for both, and each block finds its 128 rows of the
// result in its own tensor memory. A k-block of 64 then costs an SM 32 KB of shared-memory traffic
// for 128 x 256 x 64 products instead of 48 KB, which is what held the one-SM tile back, and the
// ring is six stages deep in the same space. Hand-over as above, except that both blocks' copies
// report to `full[s]` of rank 0, its commits arrive on `empty[s]` and `acc_full[a]` of both blocks,
// and both blocks' epilogue warps arrive on `acc_empty[a]` of rank 0. The blocks leave together.
#define TC2_BM 256
#define TC2_BN 256
#define TC2_THREADS 320   // warps 2-9 are the epilogue: one or two per quarter of tensor memory
#define TC2_WIDE_NKB 32
#define TC2_BAND 8          // tiles are walked in bands of 8 tile rows (2,048 rows of A)

// Where tile number `tile` lies. Within a band of TC2_BAND tile rows the row index runs fastest, so
// the pairs that work at the same time share one or two tiles of B, and a band's rows of A
// (2,048 x K) stay in L2 while all of B passes by once per band; without bands, A as a whole
// would pass by once per tile column, from DRAM as soon as it is larger than L2.
__device__ __forceinline__ void tc2_tile_origin(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band_tiles = TC2_BAND * tiles_n;
  const int band = tile / band_tiles, r = tile - band * band_tiles;
  const int rows = min(TC2_BAND, tiles_m - band * TC2_BAND);
  tm = band * TC2_BAND + r % rows;
  tn = r / rows;
}

template <int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC2_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ C,
                    int M, int N, int K, int ldc, int out_f32, int* __restrict__ err, const TcRope rp, const TcFold fd) {
  constexpr int BN = TC2_BN;
  constexpr uint32_t A_BYTES = 128 * TC_BK * 2, B_BYTES = 128 * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  volatile int* abort = (volatile int*)(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES, acc_empty0 = acc_full0 + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (M + TC2_BM - 1) / TC2_BM, tiles_n = (N + BN - 1) / BN, n_tiles = tiles_m * tiles_n;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  // A read of tensor memory waits behind the products already queued, some thousands of clocks
  // each time, so with few k-blocks to a tile four warps would take longer over a tile's epilogue
  // than the products of the next tile take: then all eight work, each on half of the columns.
  const bool wide = nkb <= TC2_WIDE_NKB || EPI == TC_EPI_RESID;     // (the residual epilogue moves five times the bytes)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, wide ? 16 : 8); }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // one warp of each block of the pair, together; both blocks get the same columns
    if (lane == 0) *tmem_slot = 0;
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                   // the other block's barriers are set up before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        int tm, tn;
        tc2_tile_origin(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * TC2_BM + (int)rank * 128, n0 = tn * BN + (int)rank * 128;
        for (int kb = 0; kb < nkb; kb++, it++) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, abort);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);     // both blocks' bytes
          uint32_t full_lead = mapa_shared(full0 + 8 * s, 0);
          uint32_t a_dst = smem_base + s * STAGE_BYTES;
          tma_load_2d_pair(a_dst, &map_a, kb * TC_BK, m0, full_lead);
          tma_load_2d_pair(a_dst + A_BYTES, &map_b, kb * TC_BK, n0, full_lead);
        }
      }
      if (*abort) {
        // copies already issued still land in this block's shared memory. Rank 0 sees them on its
        // own barriers; the other block cannot wait on those and gives its copies ample time instead.
        if (rank == 0) {
          volatile int never = 0;
          for (int j = max(0, it - STAGES); j < it; j++) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1, &never);
        } else {
          uint64_t t0 = global_ns();
          while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TC2_BM, BN);
      int it = 0, i = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, i++) {
        int a = i & 1;
        ok = mbar_wait_cluster(acc_empty0 + 8 * a, ((i >> 1) & 1) ^ 1, abort);   // both blocks have drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t acc = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < nkb; kb++, it++) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint32_t a_addr = smem_base + s * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++)
            umma_bf16_pair(acc, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc, (kb | k) ? 1u : 0u);
          umma_commit_pair(empty0 + 8 * s);
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * a);
      }
    }
  } else {
    const int q = warp & 3, c_lo = warp < 6 ? 0 : BN / 2, c_hi = wide ? c_lo + BN / 2 : BN;
    int i = 0;
    for (int tile = pair; tile < n_tiles && (wide || warp < 6); tile += n_pairs, i++) {
      int tm, tn;
      tc2_tile_origin(tile, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * TC2_BM + (int)rank * 128, n0 = tn * BN;
      int a = i & 1;
      if constexpr (EPI == TC_EPI_RESID) {
        if (!tc_epilogue_resid(tmem_base + (uint32_t)(a * BN), q, lane, m0, n0, c_lo, c_hi, (float*)C, M, N, ldc, fd,
                               (float*)(smem + STAGES * STAGE_BYTES + 256) + (warp - 2) * 1024, acc_full0 + 8 * a, (i >> 1) & 1, abort))
          break;
      } else {
        if (!mbar_wait(acc_full0 + 8 * a, (i >> 1) & 1, abort)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tc_epilogue_tile<EPI>(tmem_base + (uint32_t)(a * BN), q, lane, m0, n0, c_lo, c_hi, C, M, N, ldc, out_f32, rp, fd);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(acc_empty0 + 8 * a, 0));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                   // nothing of the other block is still on its way to this one
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort) atomicExch(err, 2);
}

template <int STAGES, int EPI>
static int tc_pair_launch(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int ldc, int out_f32,
                          int* err, cudaStream_t stream, const TcRope& rp = TcRope{}, const TcFold& fd = TcFold{}) {
  // (the residual epilogue stages its chunks through 4 KB a warp behind the barriers)
  constexpr size_t smem = STAGES * (2 * 128 * TC_BK * 2) + 1024 + 256 + (EPI == TC_EPI_RESID ? 8 * 4096 : 0);
  static int pairs = 0;                  // how many pairs of blocks the GPU holds at once
  if (!pairs) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) return SLLM_ERR_ARG - 3;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(TC2_THREADS);
    cfg.dynamicSmemBytes = smem;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<STAGES, EPI>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = sms / 2;
    }
    pairs = n < sms / 2 ? n : sms / 2;
  }
  int n_tiles = ((N + TC2_BN - 1) / TC2_BN) * ((M + TC2_BM - 1) / TC2_BM);
  dim3 grid(2 * (n_tiles < pairs ? n_tiles : pairs));
  gemm_tc_pair_kernel<STAGES, EPI><<<grid, TC2_THREADS, smem, stream>>>(ma, mb, C, M, N, K, ldc, out_f32, err, rp, fd);
  SLLM_RETURN_LAST();
}

// whether the two-SM kernel takes a product: more than one block's rows and wide enough for its tile
static bool tc_use_pair(int M, int N) {
  static int off = -1;
  if (off < 0) { const char* e = getenv("SLLM_GEMM_ONE_SM"); off = e && *e && *e != '0'; }
  return !off && M > 128 && N > 128;
}

// C[M,N] = A[M,K] B[N,K]^T. epilogue 0: C bfloat16 (or float when out_f32), row stride ldc;
// epilogue 1: C[M,N/2] = silu(gate) * up for B's rows in tiles of 16 (8 gate rows, 8 up rows);
// epilogue 2 (M > 128, N > 128 and a multiple of 32): C is the float residual stream and receives the product;
// xb[M][N] and sumsq_out[ceil(N/128)][M] receive what the product behind the following norm needs (see TcFold).
// sumsq_in (or null), n_in, width_in, eps_in: the scale owed to the rows of A (see TcFold).
// *err is set to 2 if a wait inside the kernel ran out of time.
SLLM_EXPORT int sllm_gemm_tc_fold_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                       int out_f32, int epilogue, const float* sumsq_in, int n_in, int width_in, float eps_in,
                                       const float* norm_w, void* xb, float* sumsq_out, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return SLLM_ERR_ARG;
  if (epilogue == TC_EPI_SWIGLU && ((N & 15) || out_f32)) return SLLM_ERR_ARG;
  if (epilogue != TC_EPI_SWIGLU && epilogue != TC_EPI_STORE && epilogue != TC_EPI_RESID) return SLLM_ERR_ARG;
  if (epilogue == TC_EPI_RESID && (!tc_use_pair(M, N) || (N & 31) || (ldc & 3) || !norm_w || !xb || !sumsq_out ||
                                   ((uintptr_t)C & 15) || ((uintptr_t)xb & 15) || ((uintptr_t)norm_w & 15)))
    return SLLM_ERR_ARG;
  if (sumsq_in && (n_in < 1 || width_in < 1)) return SLLM_ERR_ARG;
  const TcFold fd{sumsq_in, n_in, sumsq_in ? 1.0f / (float)width_in : 0.f, eps_in, norm_w, (bf16*)xb, sumsq_out};
  const TcRope rp{};
  CUtensorMap ma, mb;
  int big = N > 128;
  int rc = tc_make_map(&ma, A, M, K, lda, TC_BM);
  if (rc) return rc;
  if (tc_use_pair(M, N)) {
    rc = tc_make_map(&mb, B, N, K, ldb, 128);
    if (rc) return rc;
    if (epilogue == TC_EPI_SWIGLU) return tc_pair_launch<6, TC_EPI_SWIGLU>(ma, mb, C, M, N, K, ldc, 0, err, stream, rp, fd);
    if (epilogue == TC_EPI_RESID) return tc_pair_launch<6, TC_EPI_RESID>(ma, mb, C, M, N, K, ldc, 1, err, stream, rp, fd);
    return tc_pair_launch<6, TC_EPI_STORE>(ma, mb, C, M, N, K, ldc, out_f32, err, stream, rp, fd);
  }
  rc = tc_make_map(&mb, B, N, K, ldb, big ? 256 : 128);
  if (rc) return rc;
  if (epilogue == TC_EPI_SWIGLU)
    return big ? tc_launch<256, 4, TC_EPI_SWIGLU>(ma, mb, C, M, N, K, ldc, 0, err, stream, rp, fd)
               : tc_launch<128, 6, TC_EPI_SWIGLU>(ma, mb, C, M, N, K, ldc, 0, err, stream, rp, fd);
  return big ? tc_launch<256, 4, TC_EPI_STORE>(ma, mb, C, M, N, K, ldc, out_f32, err, stream, rp, fd)
             : tc_launch<128, 6, TC_EPI_STORE>(ma, mb, C, M, N, K, ldc, out_f32, err, stream, rp, fd);
}

SLLM_EXPORT int sllm_gemm_tc_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                  int out_f32, int epilogue, int* err, cudaStream_t stream) {
  if (epilogue != TC_EPI_SWIGLU && epilogue != TC_EPI_STORE) return SLLM_ERR_ARG;
  return sllm_gemm_tc_fold_bf16(A, B, C, M, N, K, lda, ldb, ldc, out_f32, epilogue, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr,
                                err, stream);
}

// C[M, (H + 2G) hd] = A[M,K] B^T with the q|k|v epilogue: rotated queries to C (bfloat16, row stride
// ldc), rotated keys and raw values to the rows' places in the cache. Pairing "half" needs the whole
// head rotated (rot == hd) and hd 64 or 128; "interleaved" any even rot. sumsq_in (or null), n_in,
// width_in, eps_in: the scale owed to the rows of A (see TcFold).
SLLM_EXPORT int sllm_gemm_tc_qkv_rope_fold_bf16(const void* A, const void* B, void* C, int M, int K, int lda, int ldb, int ldc,
                                                const int* tok_pos, const int* tok_seq, const int* block_table, int max_pages,
                                                const void* cos_sin, void* kpages, void* vpages, int H, int G, int hd, int rot,
                                                int interleaved, const float* sumsq_in, int n_in, int width_in, float eps_in,
                                                int* err, cudaStream_t stream) {
  if (M <= 0) return 0;
  int N = (H + 2 * G) * hd;
  if (K <= 0 || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15))
    return SLLM_ERR_ARG;
  if (H < 1 || G < 1 || (hd != 64 && hd != 128) || rot < 2 || rot > hd || (rot & 1) || (!interleaved && rot != hd)) return SLLM_ERR_ARG;
  if (!tok_pos || !tok_seq || !block_table || !cos_sin || !kpages || !vpages || ((uintptr_t)cos_sin & 15)) return SLLM_ERR_ARG;
  if (sumsq_in && (n_in < 1 || width_in < 1)) return SLLM_ERR_ARG;
  const TcFold fd{sumsq_in, n_in, sumsq_in ? 1.0f / (float)width_in : 0.f, eps_in, nullptr, nullptr, nullptr};
  CUtensorMap ma, mb;
  int rc = tc_make_map(&ma, A, M, K, lda, TC_BM);
  if (rc) return rc;
  TcRope rp{tok_pos, tok_seq, block_table, max_pages, (const float2*)cos_sin, (bf16*)kpages, (bf16*)vpages, H, G, hd, rot, interleaved};
  if (tc_use_pair(M, N)) {
    rc = tc_make_map(&mb, B, N, K, ldb, 128);
    if (rc) return rc;
    return tc_pair_launch<6, TC_EPI_QKV_ROPE>(ma, mb, C, M, N, K, ldc, 0, err, stream, rp, fd);
  }
  rc = tc_make_map(&mb, B, N, K, ldb, 256);
  if (rc) return rc;
  return tc_launch<256, 4, TC_EPI_QKV_ROPE>(ma, mb, C, M, N, K, ldc, 0, err, stream, rp, fd);
}

SLLM_EXPORT int sllm_gemm_tc_qkv_rope_bf16(const void* A, const void* B, void* C, int M, int K, int lda, int ldb, int ldc,
                                           const int* tok_pos, const int* tok_seq, const int* block_table, int max_pages,
                                           const void* cos_sin, void* kpages, void* vpages, int H, int G, int hd, int rot,
                                           int interleaved, int* err, cudaStream_t stream) {
  return sllm_gemm_tc_qkv_rope_fold_bf16(A, B, C, M, K, lda, ldb, ldc, tok_pos, tok_seq, block_table, max_pages, cos_sin, kpages,
                                         vpages, H, G, hd, rot, interleaved, nullptr, 0, 0, 0.f, err, stream);
}

// ------------------------------------------------------------------ few rows: the weights are the 128-row operand
// C[M,N] = A[M,K] B[N,K]^T for M <= 128 rows (a decode step of 17..128 sequences): all the time
// goes into streaming B, the weights, once. Here the roles are swapped: a block takes 128 rows of B
// as the MMA's 128-row operand and the M rows of A, padded to BT, as its columns, so the
// accumulator in tensor memory is C^T (lane = output column n, column = row m). The grid is
// (N / 128, ksplit); each block streams its 128 x K/ksplit slab of B through a deep TMA ring, and
// because weights do not depend on the kernel before, the ring is filled with them before
// griddepcontrol.wait; only then are the activations fetched. ksplit > 1 writes float partial sums
// C[ksplit][M][N] that the reader adds. EPI_SWIGLU as above (B's rows in tiles of 8 gate, 8 up).
template <int BT, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, void* __restrict__ C,
                      int M, int N, int K, int ldc, int out_f32, int* __restrict__ err) {
  constexpr uint32_t W_BYTES = 128 * TC_BK * 2, X_BYTES = BT * TC_BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr uint32_t TMEM_COLS = BT < 32 ? 32 : BT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[STAGES], empty[STAGES], acc_full
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
  volatile int* abort = (volatile int*)(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full = empty0 + 8 * STAGES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int nkb_all = (K + TC_BK - 1) / TC_BK, per = (nkb_all + gridDim.y - 1) / gridDim.y;
  const int kb0 = blockIdx.y * per, kb1 = min(nkb_all, kb0 + per), nkb = max(0, kb1 - kb0);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(acc_full, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // the first ring-full of weights goes out before the wait, their activations after it
      const int pre = min(nkb, STAGES);
      for (int i = 0; i < pre; i++) {
        mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
        tma_load_2d(smem_base + i * STAGE_BYTES, &map_w, (kb0 + i) * TC_BK, n0, full0 + 8 * i);
      }
      pdl_wait();
      for (int i = 0; i < pre; i++)
        tma_load_2d(smem_base + i * STAGE_BYTES + W_BYTES, &map_x, (kb0 + i) * TC_BK, 0, full0 + 8 * i);
      int it = pre;
      for (; it < nkb; it++) {
        int s = it % STAGES;
        if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort)) break;
        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        tma_load_2d(smem_base + s * STAGE_BYTES, &map_w, (kb0 + it) * TC_BK, n0, full0 + 8 * s);
        tma_load_2d(smem_base + s * STAGE_BYTES + W_BYTES, &map_x, (kb0 + it) * TC_BK, 0, full0 + 8 * s);
      }
      if (*abort) {
        // copies already issued still land in this block's shared memory: wait for them (bounded)
        volatile int never = 0;
        for (int j = max(0, it - STAGES); j < it; j++) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1, &never);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, BT);
      bool ok = true;
      for (int it = 0; it < nkb; it++) {
        int s = it % STAGES;
        ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t w_addr = smem_base + s * STAGE_BYTES, x_addr = w_addr + W_BYTES;
#pragma unroll
        for (int k = 0; k < TC_BK / 16; k++)
          umma_bf16(tmem_base, umma_desc_sw128(w_addr + k * 32), umma_desc_sw128(x_addr + k * 32), idesc, (it | k) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int q = warp & 3;                      // the quarter of tensor memory this warp may read
    const int n = n0 + q * 32 + lane;            // this lane's output column
    // float output: this split's own [M][N] matrix of partial sums (the only one when K is not split)
    const bool as_partial = EPI == TC_EPI_STORE && out_f32;
    float* pdst = (float*)C + (size_t)blockIdx.y * M * ldc + n;
    const int pld = ldc;
    if (nkb == 0) {
      // a split that got no k-blocks still owes the reader its (zero) partial sums
      pdl_wait();
      if (as_partial && n < N)
        for (int m = 0; m < M; m++) pdst[(size_t)m * pld] = 0.f;
    } else if (mbar_wait(acc_full, 0, abort)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      pdl_wait();        // returns at once: the activations behind the accumulator were fetched after the producer's wait
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 32) {
        if (c0 >= M) break;                      // uniform over the block
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (as_partial) {
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (n < N && c0 + j < M) pdst[(size_t)(c0 + j) * pld] = __uint_as_float(r[j]);
        } else if (EPI == TC_EPI_SWIGLU) {
          // lanes 0-7 and 16-23 hold gate rows, the lanes 8 above them the matching up rows
          int ocol = (n >> 4) * 8 + (n & 7);
          bool gate_lane = (lane & 8) == 0;
#pragma unroll
          for (int j = 0; j < 32; j++) {
            float v = __uint_as_float(r[j]);
            float u = __shfl_xor_sync(0xffffffffu, v, 8);
            if (gate_lane && n < N && c0 + j < M)
              ((bf16*)C)[(size_t)(c0 + j) * ldc + ocol] = __float2bfloat16_rn(__fdividef(v, 1.0f + __expf(-v)) * u);
          }
        } else {
          bf16* dst = (bf16*)C + n;
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (n < N && c0 + j < M) dst[(size_t)(c0 + j) * ldc] = __float2bfloat16_rn(__uint_as_float(r[j]));
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *abort) atomicExch(err, 2);
}

template <int BT, int STAGES, int EPI>
static int tc_skinny_launch(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int M, int N, int K, int ldc, int out_f32,
                            int ksplit, int* err, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (128 * TC_BK * 2 + BT * TC_BK * 2) + 1024 + 256;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_skinny_kernel<BT, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid((N + 127) / 128, ksplit);
  return (int)sllm_launch(gemm_tc_skinny_kernel<BT, STAGES, EPI>, grid, dim3(TC_THREADS), smem, stream, mw, mx, C, M, N, K, ldc,
                          out_f32, err);
}

// C[M,N] = A[M,K] B[N,K]^T for M <= 128. epilogue 0: C bfloat16, or float when out_f32; with
// ksplit > 1 (float only) C is [ksplit][M][N] partial sums. epilogue 1: C[M,N/2] = silu(gate) * up.
SLLM_EXPORT int sllm_gemm_tc_skinny_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                         int out_f32, int epilogue, int ksplit, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K <= 0 || (K & 7) || (lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return SLLM_ERR_ARG;
  if (epilogue != TC_EPI_STORE && epilogue != TC_EPI_SWIGLU) return SLLM_ERR_ARG;
  if (epilogue == TC_EPI_SWIGLU && ((N & 15) || out_f32 || ksplit != 1)) return SLLM_ERR_ARG;
  if (ksplit < 1 || ksplit > (K + TC_BK - 1) / TC_BK || (ksplit > 1 && !out_f32)) return SLLM_ERR_ARG;
  int bt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  CUtensorMap mw, mx;
  int rc = tc_make_map(&mw, B, N, K, ldb, 128);
  if (rc) return rc;
  rc = tc_make_map(&mx, A, M, K, lda, bt);
  if (rc) return rc;
#define SK_CASE(BT, ST)                                                                                                     \
  return epilogue == TC_EPI_SWIGLU ? tc_skinny_launch<BT, ST, TC_EPI_SWIGLU>(mw, mx, C, M, N, K, ldc, 0, 1, err, stream)   \
                                   : tc_skinny_launch<BT, ST, TC_EPI_STORE>(mw, mx, C, M, N, K, ldc, out_f32, ksplit, err, stream)
  if (bt == 16) { SK_CASE(16, 8); }
  if (bt == 32) { SK_CASE(32, 8); }
  if (bt == 64) { SK_CASE(64, 8); }
  SK_CASE(128, 6);
#undef SK_CASE
}

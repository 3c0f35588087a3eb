// bfloat16 kernels for the decode step (one token per sequence): everything here is bound by the
// bytes it must read once -- the weights, and the cached keys and values of the live sequences.
//
//   gemm_small_m: y[M,N] = x[M,K] W[N,K]^T for a few rows M. Each weight element is loaded from
//     HBM exactly once (16-byte loads straight into tensor-core fragments, no shared memory, two
//     register buffers used in turn so the next chunks are in flight while the current ones are
//     multiplied); the weights are the 16-row operand of mma.sync.m16n8k16 and the tokens its 8
//     columns, float accumulation. The warps of a block split K and add their partial sums in a
//     fixed order; several blocks may split K further and leave float partial sums for the reader
//     (the next norm) to add. Replaces the reference's row matmul for one token
//     (float32_ops.go:779-794) and its dense matmul for a few (float32_ops.go:462-482). An epilogue
//     can apply the SiLU gate (model_f32.go:484-490) when gate and up rows are interleaved 8 and 8.
//     An RMSNorm between two such products needs no kernel of its own: a row's 1/rms is one number,
//     so (v / rms * w) W^T = (1 / rms) * ((v * w) W^T). The product before the norm adds its result
//     to the residual stream in its epilogue, writes v * w in bfloat16 for the product after it and
//     leaves each tile's sums of v^2; the product after it adds those up, and multiplies its output
//     rows by rsqrt(sum / width + eps) (float32_ops.go:159-172 with the scale moved behind the sum
//     over k). Sums of squares, residual and scale are float.
//   attn_decode: grouped-query attention of one query per sequence over the paged cache, keys
//     split over blocks (each block streams a contiguous run of pages once and serves all query
//     heads of its key/value head), online softmax in float. The last block of a (sequence, head
//     group) to finish merges the splits. In raw mode the kernel also does the rotary step
//     (float32_ops.go:174-188) for the queries and the new key and appends key and value to the
//     cache (model_f32.go:445-448). Same mathematics as fusedAttentionHeadF32 with one query row
//     (float32_ops.go:190-235). Two kernels: attn_decode_split takes one query head at a time per
//     group of lanes; attn_decode_mma (head width 64 or 128, grouped queries or very few
//     sequences) puts the query heads of a group on the rows of mma.sync.m16n8k16 and feeds it
//     keys and values straight from the pages.
//
// All kernels here are launched with programmatic stream serialisation (see common.cuh): they may
// start while the previous kernel drains, and wait before touching what it wrote.
#include "common.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------ small-M GEMM
// Thread (g = lane/4, t = lane%4) loads 8 consecutive k of weight rows g and g+8 and of token g.
// The 8 values fill the k-slots (2t, 2t+1, 2t+8, 2t+9) of two MMAs; weights and tokens use the
// same assignment, and a sum over k does not care which slot a k sits in.
#define SM_EPI_STORE 0
#define SM_EPI_SWIGLU 1
#define SM_EPI_RESID 2

// The two halves of a norm folded into its neighbours (all pointers null: nothing folded).
struct SmFold {
  // in: the rows of x are v * w of a norm whose scale is still owed: sumsq_in[n_in][M] are partial sums of
  // v^2 over its `1 / inv_width` columns; the output rows are multiplied by rsqrt(sum * inv_width + eps)
  const float* sumsq_in;
  int n_in;
  float inv_width, eps;
  // out (SM_EPI_RESID): residual[M][ldy] += y; xb[M][N] = bfloat16(residual * norm_w); sumsq_out[tile][M] =
  // this tile's sums of residual^2
  float* residual;
  const float* norm_w;
  bf16* xb;
  float* sumsq_out;
};

__device__ __forceinline__ float ld_dep_f32(const float* p) {      // of data an earlier kernel of the stream wrote
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

template <int NT, int WARPS, int EPI, int UN, int MINB = 0>
__global__ void __launch_bounds__(WARPS * 32, MINB)
gemm_small_m_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, void* __restrict__ y, int M, int N, int K,
                    int ldx, int ldw, int ldy, int out_f32, const SmFold f) {
  __shared__ float red[WARPS][NT][4][32];
  __shared__ float row_scale[NT * 8];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  int n0 = blockIdx.x * 16;
  const bf16* w0 = W + (size_t)min(n0 + g, N - 1) * ldw;
  const bf16* w1 = W + (size_t)min(n0 + g + 8, N - 1) * ldw;
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++)
#pragma unroll
    for (int r = 0; r < 4; r++) acc[i][r] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  int nchunks = (K + 63) >> 6;
  // gridDim.y blocks share a tile's K range (their partial sums are kept apart in y); within a
  // block the warps take chunks of 64 k in turn, UN chunks in flight per warp
  int stride = gridDim.y * WARPS;
  pdl_launch_dependents();
  // Software pipeline: the weights of the next UN chunks are in flight while the current ones are
  // multiplied. The first fetch is issued before pdl_wait(): weights do not depend on earlier
  // kernels, the activations do.
  uint4 cur[UN][4], nxt[UN][4];
  auto fetch = [&](uint4 (&a)[UN][4], int c) {
#pragma unroll
    for (int u = 0; u < UN; u++) {
      int k0 = ((c + u * stride) << 6) + 8 * t, k1 = k0 + 32;
      bool ok0 = k0 < K, ok1 = k1 < K;
      a[u][0] = ok0 ? ld_stream16(w0 + k0) : zero;
      a[u][1] = ok0 ? ld_stream16(w1 + k0) : zero;
      a[u][2] = ok1 ? ld_stream16(w0 + k1) : zero;
      a[u][3] = ok1 ? ld_stream16(w1 + k1) : zero;
    }
  };
  auto multiply = [&](uint4 (&a)[UN][4], int c) {
#pragma unroll
    for (int u = 0; u < UN; u++) {
      int k0 = ((c + u * stride) << 6) + 8 * t, k1 = k0 + 32;
      bool ok0 = k0 < K, ok1 = k1 < K;
      uint4 b0[NT], b1[NT];
#pragma unroll
      for (int i = 0; i < NT; i++) {
        int tok = i * 8 + g;
        const bf16* xr = x + (size_t)tok * ldx;
        b0[i] = (tok < M && ok0) ? ld_dep16(xr + k0) : zero;
        b1[i] = (tok < M && ok1) ? ld_dep16(xr + k1) : zero;
      }
#pragma unroll
      for (int i = 0; i < NT; i++) {
        mma_16816(acc[i], a[u][0].x, a[u][1].x, a[u][0].y, a[u][1].y, b0[i].x, b0[i].y);
        mma_16816(acc[i], a[u][0].z, a[u][1].z, a[u][0].w, a[u][1].w, b0[i].z, b0[i].w);
        mma_16816(acc[i], a[u][2].x, a[u][3].x, a[u][2].y, a[u][3].y, b1[i].x, b1[i].y);
        mma_16816(acc[i], a[u][2].z, a[u][3].z, a[u][2].w, a[u][3].w, b1[i].z, b1[i].w);
      }
    }
  };
  // two register buffers used in turn (a copy between them would wait for the loads in flight)
  const int step = stride * UN;
  int c = blockIdx.y * WARPS + warp;
  fetch(cur, c);
  pdl_wait();
  // The scale each output row is owed: warp w adds up the partial sums of tokens w, w + WARPS, ... The
  // first 128 of a token's partial sums are asked for now and added after the products, so that their way
  // from L2 is not waited for.
  constexpr int TPW = (NT * 8 + WARPS - 1) / WARPS;
  float pre[TPW][4];
  if (f.sumsq_in != nullptr) {
#pragma unroll
    for (int tt = 0; tt < TPW; tt++)
#pragma unroll
      for (int k = 0; k < 4; k++) {
        int tok = warp + tt * WARPS, pt = lane + 32 * k;
        pre[tt][k] = (tok < M && pt < f.n_in) ? ld_dep_f32(f.sumsq_in + (size_t)pt * M + tok) : 0.f;
      }
  }
  // the residual values this thread will add to are asked for now as well (one output slot per thread of
  // the first NT * 128; the epilogue below walks the slots in the same order)
  float resid_pre[(NT * 128 + WARPS * 32 - 1) / (WARPS * 32)];
  if (EPI == SM_EPI_RESID) {
#pragma unroll
    for (int k = 0; k < (NT * 128 + WARPS * 32 - 1) / (WARPS * 32); k++) {
      int v = threadIdx.x + k * WARPS * 32, i = v / 128, r = (v >> 5) & 3, ln = v & 31;
      int feat = n0 + (ln >> 2) + 8 * (r >> 1), tok = 8 * i + 2 * (ln & 3) + (r & 1);
      resid_pre[k] = (v < NT * 128 && feat < N && tok < M) ? ld_dep_f32(f.residual + (size_t)tok * ldy + feat) : 0.f;
    }
  }
  while (c < nchunks) {
    fetch(nxt, c + step);
    multiply(cur, c);
    c += step;
    if (c >= nchunks) break;
    fetch(cur, c + step);
    multiply(nxt, c);
    c += step;
  }
  if (f.sumsq_in != nullptr) {
    // added in a fixed order: a lane's partial sums in turn, then a tree over the lanes
#pragma unroll
    for (int tt = 0; tt < TPW; tt++) {
      int tok = warp + tt * WARPS;
      float sq = (pre[tt][0] + pre[tt][1]) + (pre[tt][2] + pre[tt][3]);
      if (tok < M)
        for (int pt = lane + 128; pt < f.n_in; pt += 32) sq += ld_dep_f32(f.sumsq_in + (size_t)pt * M + tok);
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0 && tok < M) row_scale[tok] = rsqrtf(sq * f.inv_width + f.eps);
    }
  }
#pragma unroll
  for (int i = 0; i < NT; i++)
#pragma unroll
    for (int r = 0; r < 4; r++) red[warp][i][r][lane] = acc[i][r];
  __syncthreads();
  // acc slot r of lane (g,t): feature n0 + g + 8*(r>>1), token 8*i + 2t + (r&1)
  int v_slot = 0;
#pragma unroll
  for (int v = threadIdx.x; v < NT * 4 * 32; v += WARPS * 32, v_slot++) {
    int i = v / 128, r = (v >> 5) & 3, ln = v & 31;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) s += red[w][i][r][ln];
    const int feat = n0 + (ln >> 2) + 8 * (r >> 1), tok = 8 * i + 2 * (ln & 3) + (r & 1);
    if (f.sumsq_in != nullptr && tok < M) s *= row_scale[tok];
    if (EPI == SM_EPI_STORE) {
      if (feat < N && tok < M) {
        if (out_f32) ((float*)y)[((size_t)blockIdx.y * M + tok) * ldy + feat] = s;
        else ((bf16*)y)[(size_t)tok * ldy + feat] = __float2bfloat16_rn(s);
      }
    } else if (EPI == SM_EPI_RESID) {
      float sq = 0.f;
      if (feat < N && tok < M) {
        float* rp = f.residual + (size_t)tok * ldy + feat;
        float v = resid_pre[v_slot] + s;
        *rp = v;
        f.xb[(size_t)tok * N + feat] = __float2bfloat16_rn(v * f.norm_w[feat]);
        sq = v * v;
      }
      red[0][i][r][ln] = sq;      // slot (i, r, ln) is read by this thread only in the loop above
    } else {
      red[0][i][r][ln] = s;       // slot (i, r, ln) is read by this thread only in the loop above
    }
  }
  if (EPI == SM_EPI_RESID) {
    // a token's 16 columns of this tile lie in slots r = 2 rr + (tok & 1), ln = 4 gq + (tok % 8) / 2: added in that order
    __syncthreads();
    for (int tok = threadIdx.x; tok < NT * 8 && tok < M; tok += WARPS * 32) {
      float sq = 0.f;
#pragma unroll
      for (int rr = 0; rr < 2; rr++)
#pragma unroll
        for (int gq = 0; gq < 8; gq++) sq += red[0][tok >> 3][2 * rr + (tok & 1)][4 * gq + ((tok & 7) >> 1)];
      f.sumsq_out[(size_t)blockIdx.x * M + tok] = sq;
    }
  }
  if (EPI == SM_EPI_SWIGLU) {
    // rows g (< 8) of the tile are gate rows, rows g + 8 the matching up rows
    __syncthreads();
    for (int v = threadIdx.x; v < NT * 2 * 32; v += WARPS * 32) {
      int i = v / 64, r = (v >> 5) & 1, ln = v & 31;
      float gate = red[0][i][r][ln], up = red[0][i][r + 2][ln];
      int feat = (n0 >> 1) + (ln >> 2), tok = 8 * i + 2 * (ln & 3) + r;
      if (feat < (N >> 1) && tok < M) {
        float sg = 1.0f / (1.0f + __expf(-gate));
        ((bf16*)y)[(size_t)tok * ldy + feat] = __float2bfloat16_rn(gate * sg * up);
      }
    }
  }
}

static int sllm_sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 1;
  }
  return sms;
}

template <int NT, int WARPS, int EPI>
static int small_m_launch_w(const bf16* x, const bf16* W, void* y, int M, int N, int K, int ldx, int ldw, int ldy,
                            int out_f32, int ksplit, const SmFold& f, cudaStream_t stream) {
  dim3 grid((N + 15) / 16, ksplit);
  constexpr int UN = NT <= 2 ? 2 : 1;
  if constexpr (NT <= 2 && WARPS == 4) {
    // Blocks are equal pieces of work, so a last wave that is nearly empty costs a whole one. With one chunk
    // in flight per warp instead of two the kernel fits more blocks on an SM (seven instead of four at up to 8
    // rows; five or seven instead of three at up to 16); those forms are slower while everything is resident
    // at once and are taken where they fill their waves better: the cost of a form is its number of waves
    // times the blocks a wave holds. Measured at 8 rows: 1,024 blocks 13.4 -> 12.3 us, 1,792 blocks 43.7 ->
    // 41.3 us, 3,072 blocks 35.5 -> 34.4 us; at 16 rows: 512 blocks of K 8,192 13.1 -> 10.2 us, 1,024 blocks
    // 18.1 -> 15.4 us.
    const long long blocks = (long long)grid.x * grid.y, sms = sllm_sm_count();
    auto cost = [&](int per_sm) { const long long wave = per_sm * sms; return (blocks + wave - 1) / wave * wave; };
    const long long usual = cost(NT == 1 ? 4 : 3);
    static const bool usual_only = getenv("SLLM_SMALL_M_USUAL") != nullptr;   // for comparisons
    if (!usual_only && blocks > (NT == 1 ? 4 : 3) * sms) {
      if (cost(7) < usual && (NT == 1 || cost(7) <= cost(5)))
        return (int)sllm_launch(gemm_small_m_kernel<NT, WARPS, EPI, 1, 7>, grid, dim3(WARPS * 32), 0, stream, x, W, y, M, N, K, ldx, ldw,
                                ldy, out_f32, f);
      if constexpr (NT == 2) {
        if (cost(5) < usual)
          return (int)sllm_launch(gemm_small_m_kernel<NT, WARPS, EPI, 1, 5>, grid, dim3(WARPS * 32), 0, stream, x, W, y, M, N, K, ldx,
                                  ldw, ldy, out_f32, f);
      }
    }
  }
  return (int)sllm_launch(gemm_small_m_kernel<NT, WARPS, EPI, UN>, grid, dim3(WARPS * 32), 0, stream, x, W, y, M, N, K, ldx, ldw, ldy,
                          out_f32, f);
}

template <int NT, int EPI>
static int small_m_launch(const bf16* x, const bf16* W, void* y, int M, int N, int K, int ldx, int ldw, int ldy,
                          int out_f32, int ksplit, const SmFold& f, cudaStream_t stream) {
  if constexpr (EPI == SM_EPI_RESID) {
    // The product that feeds a folded norm cannot split K over blocks (a block must hold whole sums to add
    // them to the residual stream), so its blocks get the more warps to split K among the fewer they are:
    // about two thousand warps in all, as many loads in flight as four blocks of four had (measured: 16
    // warps win at 128 tiles, 8 at 256).
    const int tiles = (N + 15) / 16;
    if (tiles <= 160) return small_m_launch_w<NT, 16, EPI>(x, W, y, M, N, K, ldx, ldw, ldy, out_f32, ksplit, f, stream);
    if (tiles <= 384) return small_m_launch_w<NT, 8, EPI>(x, W, y, M, N, K, ldx, ldw, ldy, out_f32, ksplit, f, stream);
  }
  return small_m_launch_w<NT, 4, EPI>(x, W, y, M, N, K, ldx, ldw, ldy, out_f32, ksplit, f, stream);
}

// epilogue 0: y[M,N] in bfloat16 (or float when out_f32); epilogue 1: y[M,N/2] = silu(gate)*up with
// the rows of W interleaved 8 gate rows, 8 up rows. ksplit > 1 (float output only): K is split over
// ksplit blocks and y receives their partial sums as y[ksplit][M][ldy]; the reader adds them.
// epilogue 2 (M <= 16): y is the float residual stream [M][ldy], which receives the product; xb[M][N] and
// sumsq_out[ceil(N/16)][M] receive what the product after the following norm needs (see SmFold).
// sumsq_in (or null), n_in, width_in, eps_in: the scale owed to the rows of x (see SmFold).
SLLM_EXPORT int sllm_gemm_small_m_fold_bf16(const void* x, const void* W, void* y, int M, int N, int K, int ldx, int ldw,
                                            int ldy, int out_f32, int epilogue, int ksplit, const float* sumsq_in, int n_in,
                                            int width_in, float eps_in, const float* norm_w, void* xb, float* sumsq_out,
                                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return SLLM_ERR_ARG;
  if (epilogue == SM_EPI_SWIGLU && ((N & 15) || out_f32 || ksplit != 1)) return SLLM_ERR_ARG;
  if (epilogue == SM_EPI_RESID && (M > 16 || ksplit != 1 || !norm_w || !xb || !sumsq_out)) return SLLM_ERR_ARG;
  if (epilogue < 0 || epilogue > SM_EPI_RESID) return SLLM_ERR_ARG;
  if (ksplit < 1 || ksplit > 64 || (ksplit > 1 && !out_f32)) return SLLM_ERR_ARG;
  if (sumsq_in && (n_in < 1 || width_in < 1)) return SLLM_ERR_ARG;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  SmFold f{sumsq_in, n_in, sumsq_in ? 1.0f / (float)width_in : 0.f, eps_in, (float*)y, norm_w, (bf16*)xb, sumsq_out};
#define SM_CASE(NT)                                                                                                          \
  return epilogue == SM_EPI_SWIGLU  ? small_m_launch<NT, SM_EPI_SWIGLU>(xp, wp, y, M, N, K, ldx, ldw, ldy, 0, 1, f, stream)  \
         : epilogue == SM_EPI_RESID ? small_m_launch<(NT <= 2 ? NT : 2), SM_EPI_RESID>(xp, wp, y, M, N, K, ldx, ldw, ldy, 1, 1, f, stream) \
                                    : small_m_launch<NT, SM_EPI_STORE>(xp, wp, y, M, N, K, ldx, ldw, ldy, out_f32, ksplit, f, stream)
  if (M <= 8) { SM_CASE(1); }
  if (M <= 16) { SM_CASE(2); }
  if (M <= 32) { SM_CASE(4); }
  SM_CASE(8);
#undef SM_CASE
}

SLLM_EXPORT int sllm_gemm_small_m_bf16(const void* x, const void* W, void* y, int M, int N, int K, int ldx, int ldw,
                                       int ldy, int out_f32, int epilogue, int ksplit, cudaStream_t stream) {
  if (epilogue != SM_EPI_STORE && epilogue != SM_EPI_SWIGLU) return SLLM_ERR_ARG;
  return sllm_gemm_small_m_fold_bf16(x, W, y, M, N, K, ldx, ldw, ldy, out_f32, epilogue, ksplit, nullptr, 0, 0, 0.f, nullptr,
                                     nullptr, nullptr, stream);
}

// ------------------------------------------------------------------ decode attention, split over keys
#define AD_WARPS 4
#define AD_UN 4   // keys each lane group has in flight
#define AD_LOG2E 1.4426950408889634f
#define AD_MAX_SPLIT 64   // splits the merging block weighs with one warp pass; more are merged the slow way

struct AttnDecodeArgs {
  const bf16* q;        // [B, q_ld] rotated queries of this step, head h at columns h*HD
  int q_ld;
  const int* seq_pos0;  // [B] position of the query = number of keys cached before this step
  const int* block_table;
  int max_pages;
  const bf16* kpages;   // [pages][G][PAGE][HD]
  const bf16* vpages;
  float* part;          // [B][H][n_split][HD + 2]: unnormalised sum, running max (log2 units), running sum
  int H, G, window, n_split;
  float scale;
  bf16* out;            // [B, H*HD]; written by this kernel only when `tickets` is given
  int* tickets;         // [B*G] zero before the first launch, or null: a separate kernel merges the splits
  // raw mode (cs != null): `q` is the step's unrotated [q heads | k heads | v heads] rows; the kernel
  // rotates the queries itself and, when write_kv is set, rotates the new key, stores it and the new
  // value at position seq_pos0[b] of the cache and uses them -- no separate rotary kernel
  const float2* cs;     // [positions][rot/2] (cos, sin)
  int rot, interleaved, write_kv;
  int late;             // no key is asked for before the wait for the kernel in front (for comparisons)
};

// Eight consecutive dims [d0, d0+8) of a head's raw row, rotated for the position whose table row
// is `csr`, rounded to bfloat16 as the rotary kernel would store them.
__device__ __forceinline__ void rope8_raw(const bf16* head, int d0, int rot, int interleaved, const float2* csr, float (&out)[8]) {
  uint4 raw = ld_dep16(head + d0);
  const bf16* e = (const bf16*)&raw;
  float x[8];
#pragma unroll
  for (int j = 0; j < 8; j++) x[j] = __bfloat162float(e[j]);
  if (d0 >= rot) {
#pragma unroll
    for (int j = 0; j < 8; j++) out[j] = x[j];
    return;
  }
  int half = rot >> 1;
  if (interleaved) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float2 c = csr[(d0 >> 1) + j];
      out[2 * j] = x[2 * j] * c.x - x[2 * j + 1] * c.y;
      out[2 * j + 1] = x[2 * j] * c.y + x[2 * j + 1] * c.x;
    }
  } else {
    bool first = d0 < half;
    uint4 praw = ld_dep16(head + (first ? d0 + half : d0 - half));
    const bf16* pe = (const bf16*)&praw;
    const float2* c0 = csr + (first ? d0 : d0 - half);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      float y = __bfloat162float(pe[j]);
      float2 c = c0[j];
      out[j] = first ? x[j] * c.x - y * c.y : y * c.y + x[j] * c.x;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; j++) out[j] = __bfloat162float(__float2bfloat16_rn(out[j]));
}

// The block that finishes last among the splits of a (sequence, key/value head) merges them: every
// block publishes its partial results, then takes a ticket; nobody waits for anybody.
__device__ __forceinline__ void ad_ticket_merge(const AttnDecodeArgs& p, int b, int g, int nrep, int HD) {
  if (p.tickets == nullptr || p.n_split == 1) return;     // one split: its block wrote the output itself
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = p.tickets + (size_t)b * p.G + g;
    int t = atomicAdd(tk, 1);
    s_last = (t == p.n_split - 1);
    if (s_last) *tk = 0;                       // all splits have drawn: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (p.n_split > 8 && p.n_split <= AD_MAX_SPLIT) {
    // many splits, eight heads at a time: a warp per head weighs the splits (lanes over splits), then every
    // thread adds one output element over the splits with loads that do not depend on each other
    __shared__ float sm_c[8][AD_MAX_SPLIT];
    __shared__ float sm_l[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h0 = 0; h0 < nrep; h0 += 8) {
      const int nh = min(8, nrep - h0);
      for (int r = warp; r < nh; r += AD_WARPS) {
        const float* src = p.part + ((size_t)b * p.H + g * nrep + h0 + r) * p.n_split * (HD + 2) + HD;
        float ms[AD_MAX_SPLIT / 32], ls[AD_MAX_SPLIT / 32], mn = -INFINITY;
#pragma unroll
        for (int i = 0; i < AD_MAX_SPLIT / 32; i++) {
          int s2 = lane + 32 * i;
          ms[i] = s2 < p.n_split ? __ldcg(src + (size_t)s2 * (HD + 2)) : -INFINITY;
          ls[i] = s2 < p.n_split ? __ldcg(src + (size_t)s2 * (HD + 2) + 1) : 0.f;
          mn = fmaxf(mn, ms[i]);
        }
        mn = warp_max(mn);
        float lsum = 0.f;
#pragma unroll
        for (int i = 0; i < AD_MAX_SPLIT / 32; i++) {
          float c = (mn == -INFINITY || ms[i] == -INFINITY) ? 0.f : exp2f(ms[i] - mn);
          sm_c[r][lane + 32 * i] = c;
          lsum += ls[i] * c;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) sm_l[r] = lsum;
      }
      __syncthreads();
      for (int v = threadIdx.x; v < nh * HD; v += AD_WARPS * 32) {
        int r = v / HD, dd = v % HD, h = g * nrep + h0 + r;
        const float* src = p.part + ((size_t)b * p.H + h) * p.n_split * (HD + 2) + dd;
        float a = 0.f;
#pragma unroll 8
        for (int s2 = 0; s2 < p.n_split; s2++) a += __ldcg(src + (size_t)s2 * (HD + 2)) * sm_c[r][s2];
        float ls = sm_l[r];
        p.out[((size_t)b * p.H + h) * HD + dd] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
      }
      __syncthreads();
    }
    return;
  }
  for (int v = threadIdx.x; v < nrep * HD; v += AD_WARPS * 32) {
    int h = g * nrep + v / HD, dd = v % HD;
    const float* src = p.part + ((size_t)b * p.H + h) * p.n_split * (HD + 2);
    float mn = -INFINITY;
    for (int s2 = 0; s2 < p.n_split; s2++) mn = fmaxf(mn, __ldcg(src + (size_t)s2 * (HD + 2) + HD));
    float a = 0.f, ls = 0.f;
    for (int s2 = 0; s2 < p.n_split; s2++) {
      const float* ps = src + (size_t)s2 * (HD + 2);
      float ms = __ldcg(ps + HD);
      float c = (mn == -INFINITY || ms == -INFINITY) ? 0.f : exp2f(ms - mn);
      a += __ldcg(ps + dd) * c;
      ls += __ldcg(ps + HD + 1) * c;
    }
    p.out[((size_t)b * p.H + h) * HD + dd] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
  }
}

template <bool FIRST, typename T>
__device__ __forceinline__ T& ad_pick(T& a, T& b) {
  if constexpr (FIRST) return a;
  else return b;
}

template <int HD, int NREP, bool RAW, bool EARLY>
__global__ void __launch_bounds__(AD_WARPS * 32, NREP == 1 ? 7 : 1) attn_decode_split_kernel(AttnDecodeArgs p) {
  constexpr int LPK = HD / 8;        // lanes that share one key (8 dims = 16 bytes each)
  constexpr int KPW = 32 / LPK;      // keys a warp reads per load
  __shared__ float sm_acc[AD_WARPS][NREP][HD];
  __shared__ float sm_ml[AD_WARPS][NREP][2];
  pdl_launch_dependents();
  if (!RAW) pdl_wait();        // given finished queries, the kernel in front may have written any of its inputs
  int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int slot = lane / LPK, dl = (lane % LPK) * 8;
  int pos = p.seq_pos0[b];
  int k_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  int pb = k_begin / SLLM_PAGE, pe = pos / SLLM_PAGE;
  int pps = (pe - pb + 1 + p.n_split - 1) / p.n_split;
  int p0 = pb + split * pps, p1 = min(pe + 1, p0 + pps);
  int k_lo = max(k_begin, p0 * SLLM_PAGE), k_hi = min(pos + 1, p1 * SLLM_PAGE);
  const int* bt = p.block_table + (size_t)b * p.max_pages;
  int nrep = p.H / p.G;
  // raw mode: the key at the query's own position is not in the cache yet; the block whose range
  // holds it takes it from the step's raw row after the cached keys
  const bool has_new = RAW && p.write_kv && pos >= k_lo && pos < k_hi;
  const int k_end = has_new ? pos : k_hi;

  auto fetch = [&](uint4 (&kr)[AD_UN], uint4 (&vr)[AD_UN], bool (&ok)[AD_UN], int kb) {
#pragma unroll
    for (int u = 0; u < AD_UN; u++) {
      int key = kb + u * KPW + slot;
      ok[u] = key < k_end;
      int kk = ok[u] ? key : k_lo;
      int page = bt[kk / SLLM_PAGE];
      size_t off = (((size_t)page * p.G + g) * SLLM_PAGE + (kk % SLLM_PAGE)) * HD + dl;
      kr[u] = ld_dep16_stream(p.kpages + off);
      vr[u] = ld_dep16_stream(p.vpages + off);
    }
  };
  // The warp's first keys are asked for before the wait for the kernel in front (whose output is this step's
  // q, k and v): keys before the query's position were cached by earlier steps, and a step's first kernel
  // is launched the ordinary way, after everything before it. The sequence's length and page numbers are
  // step inputs, copied in before the step. Not so the key at the query's own position.
  // (EARLY is chosen where all blocks are resident at once: there nothing else hides that chain of loads;
  // the registers it costs are spilled over the wait.)
  const int kb0 = k_lo + warp * KPW * AD_UN;
  const bool early = EARLY && kb0 < k_end && kb0 + KPW * AD_UN <= pos;
  uint4 kr0[AD_UN], vr0[AD_UN];          // the loop's own buffers when EARLY (else unused: it declares its own)
  bool ok0[AD_UN];
  if constexpr (EARLY) {
    if (early) fetch(kr0, vr0, ok0, kb0);
  }
  if (RAW) pdl_wait();

  for (int r0 = 0; r0 < nrep; r0 += NREP) {
    float q[NREP][8], acc[NREP][8], m[NREP], l[NREP];
#pragma unroll
    for (int r = 0; r < NREP; r++) {
      int h = g * nrep + r0 + r;
      if (RAW) {
        float qr[8];
        rope8_raw(p.q + (size_t)b * p.q_ld + (size_t)h * HD, dl, p.rot, p.interleaved, p.cs + (size_t)pos * (p.rot >> 1), qr);
#pragma unroll
        for (int j = 0; j < 8; j++) { q[r][j] = qr[j] * (p.scale * AD_LOG2E); acc[r][j] = 0.f; }
      } else {
        uint4 raw = ld_dep16(p.q + (size_t)b * p.q_ld + (size_t)h * HD + dl);
        const bf16* e = (const bf16*)&raw;
#pragma unroll
        for (int j = 0; j < 8; j++) { q[r][j] = __bfloat162float(e[j]) * (p.scale * AD_LOG2E); acc[r][j] = 0.f; }
      }
      m[r] = -INFINITY;
      l[r] = 0.f;
    }
    for (int kb = kb0; kb < k_end; kb += AD_WARPS * KPW * AD_UN) {
      uint4 kr1[AD_UN], vr1[AD_UN];
      bool ok1[AD_UN];
      uint4 (&kr)[AD_UN] = ad_pick<EARLY>(kr0, kr1);
      uint4 (&vr)[AD_UN] = ad_pick<EARLY>(vr0, vr1);
      bool (&ok)[AD_UN] = ad_pick<EARLY>(ok0, ok1);
      if (!(EARLY && early && r0 == 0 && kb == kb0)) fetch(kr, vr, ok, kb);
      float s[AD_UN][NREP];
#pragma unroll
      for (int u = 0; u < AD_UN; u++) {
        const bf16* ke = (const bf16*)&kr[u];
        float kf[8];
#pragma unroll
        for (int j = 0; j < 8; j++) kf[j] = __bfloat162float(ke[j]);
#pragma unroll
        for (int r = 0; r < NREP; r++) {
          float d = 0.f;
#pragma unroll
          for (int j = 0; j < 8; j++) d = fmaf(q[r][j], kf[j], d);
#pragma unroll
          for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          s[u][r] = ok[u] ? d : -INFINITY;
        }
      }
#pragma unroll
      for (int r = 0; r < NREP; r++) {
        float m_new = m[r];
#pragma unroll
        for (int u = 0; u < AD_UN; u++) m_new = fmaxf(m_new, s[u][r]);
        if (m_new == -INFINITY) continue;
        float corr = exp2f(m[r] - m_new);
        m[r] = m_new;
        float lsum = l[r] * corr;
#pragma unroll
        for (int j = 0; j < 8; j++) acc[r][j] *= corr;
#pragma unroll
        for (int u = 0; u < AD_UN; u++) {
          float pr = exp2f(s[u][r] - m_new);
          lsum += pr;
          const bf16* ve = (const bf16*)&vr[u];
#pragma unroll
          for (int j = 0; j < 8; j++) acc[r][j] = fmaf(pr, __bfloat162float(ve[j]), acc[r][j]);
        }
        l[r] = lsum;
      }
    }
    if (has_new) {
      // this step's own key and value: rotate, round, store at their place in the cache, use
      bool mine = warp == 0 && slot == 0;
      float kn[8], vn[8];
#pragma unroll
      for (int j = 0; j < 8; j++) kn[j] = vn[j] = 0.f;
      if (mine) {
        const bf16* rowp = p.q + (size_t)b * p.q_ld;
        rope8_raw(rowp + (size_t)(p.H + g) * HD, dl, p.rot, p.interleaved, p.cs + (size_t)pos * (p.rot >> 1), kn);
        uint4 vraw = ld_dep16(rowp + (size_t)(p.H + p.G + g) * HD + dl);
        const bf16* ve = (const bf16*)&vraw;
#pragma unroll
        for (int j = 0; j < 8; j++) vn[j] = __bfloat162float(ve[j]);
        if (r0 == 0) {
          size_t off = (((size_t)bt[pos / SLLM_PAGE] * p.G + g) * SLLM_PAGE + (pos % SLLM_PAGE)) * HD + dl;
          uint4 kraw;
          __nv_bfloat162* kp2 = (__nv_bfloat162*)&kraw;
#pragma unroll
          for (int j = 0; j < 4; j++) kp2[j] = __floats2bfloat162_rn(kn[2 * j], kn[2 * j + 1]);
          *(uint4*)(const_cast<bf16*>(p.kpages) + off) = kraw;
          *(uint4*)(const_cast<bf16*>(p.vpages) + off) = vraw;
        }
      }
#pragma unroll
      for (int r = 0; r < NREP; r++) {
        float d = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) d = fmaf(q[r][j], kn[j], d);
#pragma unroll
        for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (!mine) continue;
        float m_new = fmaxf(m[r], d);
        float corr = exp2f(m[r] - m_new), pr = exp2f(d - m_new);
        m[r] = m_new;
        l[r] = l[r] * corr + pr;
#pragma unroll
        for (int j = 0; j < 8; j++) acc[r][j] = fmaf(pr, vn[j], acc[r][j] * corr);
      }
    }
    // merge the key slots of the warp, then the warps
#pragma unroll
    for (int r = 0; r < NREP; r++) {
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) {
        float mo = __shfl_xor_sync(0xffffffffu, m[r], o), lo = __shfl_xor_sync(0xffffffffu, l[r], o);
        float mn = fmaxf(m[r], mo);
        float c1 = mn == -INFINITY ? 0.f : exp2f(m[r] - mn), c2 = mn == -INFINITY ? 0.f : exp2f(mo - mn);
        l[r] = l[r] * c1 + lo * c2;
        m[r] = mn;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float ao = __shfl_xor_sync(0xffffffffu, acc[r][j], o);
          acc[r][j] = acc[r][j] * c1 + ao * c2;
        }
      }
      if (lane < LPK) {
#pragma unroll
        for (int j = 0; j < 8; j++) sm_acc[warp][r][dl + j] = acc[r][j];
        if (lane == 0) { sm_ml[warp][r][0] = m[r]; sm_ml[warp][r][1] = l[r]; }
      }
    }
    __syncthreads();
    for (int v = threadIdx.x; v < NREP * HD; v += AD_WARPS * 32) {
      int r = v / HD, dd = v % HD;
      float mn = -INFINITY;
#pragma unroll
      for (int w = 0; w < AD_WARPS; w++) mn = fmaxf(mn, sm_ml[w][r][0]);
      float a = 0.f, ls = 0.f;
#pragma unroll
      for (int w = 0; w < AD_WARPS; w++) {
        float c = mn == -INFINITY ? 0.f : exp2f(sm_ml[w][r][0] - mn);
        a += sm_acc[w][r][dd] * c;
        ls += sm_ml[w][r][1] * c;
      }
      int h = g * nrep + r0 + r;
      float* dst = p.part + (((size_t)b * p.H + h) * p.n_split + split) * (HD + 2);
      dst[dd] = a;
      if (dd == 0) { dst[HD] = mn; dst[HD + 1] = ls; }
    }
    __syncthreads();
  }
  if (p.tickets == nullptr) return;
  // The block that finishes last among the splits of this (sequence, key/value head) merges them:
  // every block publishes its partial results, then takes a ticket; nobody waits for anybody.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = p.tickets + (size_t)b * p.G + g;
    int t = atomicAdd(tk, 1);
    s_last = (t == p.n_split - 1);
    if (s_last) *tk = 0;                       // all splits have drawn: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int v = threadIdx.x; v < nrep * HD; v += AD_WARPS * 32) {
    int h = g * nrep + v / HD, dd = v % HD;
    const float* src = p.part + ((size_t)b * p.H + h) * p.n_split * (HD + 2);
    float mn = -INFINITY;
    for (int s2 = 0; s2 < p.n_split; s2++) mn = fmaxf(mn, __ldcg(src + (size_t)s2 * (HD + 2) + HD));
    float a = 0.f, ls = 0.f;
    for (int s2 = 0; s2 < p.n_split; s2++) {
      const float* ps = src + (size_t)s2 * (HD + 2);
      float ms = __ldcg(ps + HD);
      float c = (mn == -INFINITY || ms == -INFINITY) ? 0.f : exp2f(ms - mn);
      a += __ldcg(ps + dd) * c;
      ls += __ldcg(ps + HD + 1) * c;
    }
    p.out[((size_t)b * p.H + h) * HD + dd] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
  }
}

// Grouped-query variant on the tensor cores (mma.sync.m16n8k16), for 2 or more query heads per
// key/value head: the heads of the group are the 16 rows of the MMA, a tile of 16 keys its
// columns. Lane (n = lane/4, t = lane%4) loads keys and values straight from the pages into
// fragments with 16-byte loads, no shared memory:
//   scores: B operand = K; the lane loads dims [(4j+t)*8, +8) of key n; those 8 dims fill the k-slots
//     (2t, 2t+1, 2t+8, 2t+9) of two MMAs and the query fragments use the same assignment.
//   output: A operand = the probabilities, whose layout is the one the score MMAs left them in;
//     B operand = V, which the MMA wants as pairs of keys for one dim: the lane loads dims
//     [n*8, +8) of keys 2t, 2t+1, 2t+8, 2t+9 and pairs them up with byte permutes. Column n of
//     output tile jt is dim n*8 + jt.
// UP: rows 8..15 carry heads too (more than 8 heads per group). The maximum is kept per row over
// the four lanes that share it, and the running output is rescaled only when some row's grew.
template <int HD, bool UP, bool RAW>
__global__ void __launch_bounds__(AD_WARPS * 32) attn_decode_mma_kernel(AttnDecodeArgs p) {
  constexpr int ROWS = UP ? 16 : 8;
  constexpr int CH = HD / 8;       // 16-byte chunks of a head row
  constexpr int NJ = HD / 32;      // pairs of k-steps of the score product
  constexpr int NC = HD / 64;      // 64-dim column blocks of the output
  __shared__ __align__(16) bf16 sm_q[ROWS][HD];
  __shared__ float sm_acc[AD_WARPS][ROWS][HD + 1];
  __shared__ float sm_ml[AD_WARPS][ROWS][2];
  pdl_launch_dependents();
  if (!RAW) pdl_wait();        // given finished queries, the kernel in front may have written any of its inputs
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = lane >> 2, t = lane & 3;
  const int pos = p.seq_pos0[b];
  const int k_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int pb = k_begin / SLLM_PAGE, pe = pos / SLLM_PAGE;
  const int pps = (pe - pb + 1 + p.n_split - 1) / p.n_split;
  const int p0 = pb + split * pps, p1 = min(pe + 1, p0 + pps);
  const int k_lo = max(k_begin, p0 * SLLM_PAGE), k_hi = min(pos + 1, p1 * SLLM_PAGE);
  const int* bt = p.block_table + (size_t)b * p.max_pages;
  const int nrep = p.H / p.G;
  const bf16* rowp = p.q + (size_t)b * p.q_ld;
  const float2* csr = RAW ? p.cs + (size_t)pos * (p.rot >> 1) : nullptr;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const float sc = p.scale * AD_LOG2E;

  auto fetch = [&](uint4 (&kr)[2][NJ], uint4 (&vr)[4][NC], int base) {
    const size_t row0 = ((size_t)bt[base / SLLM_PAGE] * p.G + g) * SLLM_PAGE + (base % SLLM_PAGE);
    const bf16* kp = p.kpages + row0 * HD;
    const bf16* vp = p.vpages + row0 * HD;
#pragma unroll
    for (int u = 0; u < 2; u++) {
      int key = base + u * 8 + n;
      bool ok = key >= k_lo && key < k_hi;
#pragma unroll
      for (int j = 0; j < NJ; j++) kr[u][j] = ok ? ld_dep16_stream(kp + (size_t)(u * 8 + n) * HD + (j * 4 + t) * 8) : zero;
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int kk = 2 * t + (i & 1) + (i >> 1) * 8;
      bool ok = base + kk >= k_lo && base + kk < k_hi;
#pragma unroll
      for (int c = 0; c < NC; c++) vr[i][c] = ok ? ld_dep16_stream(vp + (size_t)kk * HD + (c * 8 + n) * 8) : zero;
    }
  };
  // In raw mode (the kernel is part of a model step) the warp's first tile of keys is asked for before the
  // wait for the kernel in front, as in attn_decode_split_kernel: keys before the query's position were
  // cached by earlier steps. It pays where the blocks are few (one head per key/value head and few
  // sequences); with grouped queries it changed nothing.
  constexpr int STEP = AD_WARPS * 16;
  const int base0 = (k_lo & ~15) + warp * 16;
  const bool early = RAW && !p.late && base0 < k_hi && base0 + 16 <= pos;
  uint4 ka[2][NJ], va[4][NC];
  if (early) fetch(ka, va, base0);
  if (RAW) pdl_wait();

  // raw mode: the block whose range holds the query's own position rotates the new key and appends
  // key and value to the cache; after the barrier below they are cached keys like the others
  if (RAW && p.write_kv && pos >= k_lo && pos < k_hi && threadIdx.x < CH) {
    int dl = threadIdx.x * 8;
    float kn[8];
    rope8_raw(rowp + (size_t)(p.H + g) * HD, dl, p.rot, p.interleaved, csr, kn);
    uint4 vraw = ld_dep16(rowp + (size_t)(p.H + p.G + g) * HD + dl);
    uint4 kraw;
    __nv_bfloat162* kp2 = (__nv_bfloat162*)&kraw;
#pragma unroll
    for (int j = 0; j < 4; j++) kp2[j] = __floats2bfloat162_rn(kn[2 * j], kn[2 * j + 1]);
    size_t off = (((size_t)bt[pos / SLLM_PAGE] * p.G + g) * SLLM_PAGE + (pos % SLLM_PAGE)) * HD + dl;
    *(uint4*)(const_cast<bf16*>(p.kpages) + off) = kraw;
    *(uint4*)(const_cast<bf16*>(p.vpages) + off) = vraw;
  }

  for (int r0 = 0; r0 < nrep; r0 += ROWS) {
    for (int i = threadIdx.x; i < ROWS * CH; i += AD_WARPS * 32) {
      int r = i / CH, dl = (i % CH) * 8;
      uint4 val = zero;
      if (r0 + r < nrep) {
        const bf16* head = rowp + (size_t)(g * nrep + r0 + r) * HD;
        if (RAW) {
          float qr[8];
          rope8_raw(head, dl, p.rot, p.interleaved, csr, qr);
          __nv_bfloat162* q2 = (__nv_bfloat162*)&val;
#pragma unroll
          for (int j = 0; j < 4; j++) q2[j] = __floats2bfloat162_rn(qr[2 * j], qr[2 * j + 1]);
        } else {
          val = ld_dep16(head + dl);
        }
      }
      *(uint4*)&sm_q[r][dl] = val;
    }
    __syncthreads();
    uint32_t qa[2 * NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
      uint4 lo = *(const uint4*)&sm_q[n][(j * 4 + t) * 8];
      uint4 hi = UP ? *(const uint4*)&sm_q[UP ? n + 8 : n][(j * 4 + t) * 8] : zero;
      qa[2 * j][0] = lo.x; qa[2 * j][1] = hi.x; qa[2 * j][2] = lo.y; qa[2 * j][3] = hi.y;
      qa[2 * j + 1][0] = lo.z; qa[2 * j + 1][1] = hi.z; qa[2 * j + 1][2] = lo.w; qa[2 * j + 1][3] = hi.w;
    }
    float o[NC * 8][4];
#pragma unroll
    for (int i = 0; i < NC * 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    auto attend = [&](uint4 (&kr)[2][NJ], uint4 (&vr)[4][NC], int base) {
      float s[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        s[u][0] = s[u][1] = s[u][2] = s[u][3] = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; j++) {
          mma_16816(s[u], qa[2 * j][0], qa[2 * j][1], qa[2 * j][2], qa[2 * j][3], kr[u][j].x, kr[u][j].y);
          mma_16816(s[u], qa[2 * j + 1][0], qa[2 * j + 1][1], qa[2 * j + 1][2], qa[2 * j + 1][3], kr[u][j].z, kr[u][j].w);
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {
          int key = base + u * 8 + 2 * t + (e & 1);
          s[u][e] = (key >= k_lo && key < k_hi) ? s[u][e] * sc : -INFINITY;
        }
      }
      float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      float mx1 = UP ? fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3])) : -INFINITY;
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      if (UP) {
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      }
      if (__any_sync(0xffffffffu, mx0 > m0 || (UP && mx1 > m1))) {
        float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        float c0 = n0 == -INFINITY ? 1.f : exp2f(m0 - n0), c1 = n1 == -INFINITY ? 1.f : exp2f(m1 - n1);
        m0 = n0; m1 = n1;
        l0 *= c0; l1 *= c1;
#pragma unroll
        for (int i = 0; i < NC * 8; i++) {
          o[i][0] *= c0; o[i][1] *= c0;
          if (UP) { o[i][2] *= c1; o[i][3] *= c1; }
        }
      }
      const float u0 = m0 == -INFINITY ? 0.f : m0, u1 = m1 == -INFINITY ? 0.f : m1;
      float pr[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        pr[u][0] = exp2f(s[u][0] - u0); pr[u][1] = exp2f(s[u][1] - u0);
        pr[u][2] = UP ? exp2f(s[u][2] - u1) : 0.f; pr[u][3] = UP ? exp2f(s[u][3] - u1) : 0.f;
      }
      l0 += (pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]);
      if (UP) l1 += (pr[0][2] + pr[0][3]) + (pr[1][2] + pr[1][3]);
      __nv_bfloat162 h0 = __floats2bfloat162_rn(pr[0][0], pr[0][1]), h1 = __floats2bfloat162_rn(pr[0][2], pr[0][3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(pr[1][0], pr[1][1]), h3 = __floats2bfloat162_rn(pr[1][2], pr[1][3]);
      const uint32_t pa0 = *(uint32_t*)&h0, pa1 = UP ? *(uint32_t*)&h1 : 0u, pa2 = *(uint32_t*)&h2, pa3 = UP ? *(uint32_t*)&h3 : 0u;
#pragma unroll
      for (int c = 0; c < NC; c++) {
        const uint32_t* va = (const uint32_t*)&vr[0][c];
        const uint32_t* vb = (const uint32_t*)&vr[1][c];
        const uint32_t* vc = (const uint32_t*)&vr[2][c];
        const uint32_t* vd = (const uint32_t*)&vr[3][c];
#pragma unroll
        for (int jt = 0; jt < 8; jt++) {
          const uint32_t sel = (jt & 1) ? 0x7632u : 0x5410u;
          uint32_t b0 = __byte_perm(va[jt >> 1], vb[jt >> 1], sel), b1 = __byte_perm(vc[jt >> 1], vd[jt >> 1], sel);
          mma_16816(o[c * 8 + jt], pa0, pa1, pa2, pa3, b0, b1);
        }
      }
    };
    // a warp takes every AD_WARPS-th tile of 16 keys; two register buffers used in turn, so the next
    // tile's keys and values are in flight while the current tile is multiplied
    int base = base0;
    const bool have = early && r0 == 0;        // the first tile is here already
    if constexpr (HD >= 128) {
      // two register buffers used in turn: the next tile is in flight while this one is multiplied.
      // (At width 64 a tile is too small for that to pay for the registers.)
      uint4 kb[2][NJ], vb[4][NC];
      if (base < k_hi && !have) fetch(ka, va, base);
      while (base < k_hi) {
        if (base + STEP < k_hi) fetch(kb, vb, base + STEP);
        attend(ka, va, base);
        base += STEP;
        if (base >= k_hi) break;
        if (base + STEP < k_hi) fetch(ka, va, base + STEP);
        attend(kb, vb, base);
        base += STEP;
      }
    } else {
      for (; base < k_hi; base += STEP) {
        if (!(have && base == base0)) fetch(ka, va, base);
        attend(ka, va, base);
      }
    }
    // the four lanes of a row hold different keys' shares of the sum; then the warps are merged
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    if (UP) {
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
      for (int jt = 0; jt < 8; jt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          int d = (c * 8 + 2 * t + e) * 8 + jt;
          sm_acc[warp][n][d] = o[c * 8 + jt][e];
          if (UP) sm_acc[warp][UP ? n + 8 : n][d] = o[c * 8 + jt][2 + e];
        }
    if (t == 0) {
      sm_ml[warp][n][0] = m0; sm_ml[warp][n][1] = l0;
      if (UP) { sm_ml[warp][UP ? n + 8 : n][0] = m1; sm_ml[warp][UP ? n + 8 : n][1] = l1; }
    }
    __syncthreads();
    const int rows = min(ROWS, nrep - r0);
    for (int v = threadIdx.x; v < rows * HD; v += AD_WARPS * 32) {
      int r = v / HD, dd = v % HD;
      float mn = -INFINITY;
#pragma unroll
      for (int w = 0; w < AD_WARPS; w++) mn = fmaxf(mn, sm_ml[w][r][0]);
      float a = 0.f, ls = 0.f;
#pragma unroll
      for (int w = 0; w < AD_WARPS; w++) {
        float c = mn == -INFINITY ? 0.f : exp2f(sm_ml[w][r][0] - mn);
        a += sm_acc[w][r][dd] * c;
        ls += sm_ml[w][r][1] * c;
      }
      if (p.n_split == 1 && p.tickets != nullptr) {        // nothing to merge with: this is the result
        p.out[((size_t)b * p.H + g * nrep + r0 + r) * HD + dd] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
        continue;
      }
      float* dst = p.part + (((size_t)b * p.H + g * nrep + r0 + r) * p.n_split + split) * (HD + 2);
      dst[dd] = a;
      if (dd == 0) { dst[HD] = mn; dst[HD + 1] = ls; }
    }
    __syncthreads();
  }
  ad_ticket_merge(p, b, g, nrep, HD);
}

// out[b, h*HD + d] = sum_s acc_s[d] 2^(m_s - M) / sum_s l_s 2^(m_s - M)
__global__ void attn_decode_merge_kernel(const float* __restrict__ part, bf16* __restrict__ out, int H, int HD,
                                         int n_split) {
  pdl_launch_dependents();
  pdl_wait();
  int h = blockIdx.x, b = blockIdx.y;
  const float* src = part + ((size_t)b * H + h) * n_split * (HD + 2);
  float mn = -INFINITY;
  for (int s = 0; s < n_split; s++) mn = fmaxf(mn, ld_dep(src + (size_t)s * (HD + 2) + HD));
  for (int dd = threadIdx.x; dd < HD; dd += blockDim.x) {
    float a = 0.f, ls = 0.f;
    for (int s = 0; s < n_split; s++) {
      const float* ps = src + (size_t)s * (HD + 2);
      float ms = ld_dep(ps + HD);
      float c = (mn == -INFINITY || ms == -INFINITY) ? 0.f : exp2f(ms - mn);
      a += ld_dep(ps + dd) * c;
      ls += ld_dep(ps + HD + 1) * c;
    }
    out[((size_t)b * H + h) * HD + dd] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
  }
}

// Which of the two kernels serves a shape: the tensor-core one for grouped queries, and also for
// one head per group while there are so few (sequence, head) pairs that its shorter chain of
// instructions per key decides (measured: 10.7 against 15.9 us at 32 pairs, even at 256).
static bool attn_decode_uses_mma(int B, int H, int G, int hd) {
  if (hd != 64 && hd != 128) return false;
  return H >= 2 * G || (long long)B * G <= 64;
}
SLLM_EXPORT int sllm_attn_decode_uses_mma(int B, int H, int G, int hd) { return attn_decode_uses_mma(B, H, G, hd) ? 1 : 0; }

template <int HD>
static int attn_decode_launch(const AttnDecodeArgs& a, bf16* out, int B, cudaStream_t stream) {
  dim3 grid(a.n_split, a.G, B);
  int nrep = a.H / a.G;
  cudaError_t e;
  if constexpr (HD == 64 || HD == 128) {
    static const bool scalar_only = getenv("SLLM_DECODE_SCALAR") != nullptr;   // for comparisons
    if (attn_decode_uses_mma(B, a.H, a.G, HD) && !scalar_only) {
      bool up = nrep > 8;
#define AD_MMA(UPV, RAWV) sllm_launch(attn_decode_mma_kernel<HD, UPV, RAWV>, grid, dim3(AD_WARPS * 32), 0, stream, a)
      if (a.cs != nullptr) e = up ? AD_MMA(true, true) : AD_MMA(false, true);
      else e = up ? AD_MMA(true, false) : AD_MMA(false, false);
#undef AD_MMA
      if (e != cudaSuccess || a.tickets != nullptr) return (int)e;
      return (int)sllm_launch(attn_decode_merge_kernel, dim3(a.H, B), dim3(HD), 0, stream, (const float*)a.part, out, a.H,
                              HD, a.n_split);
    }
  }
  if (a.cs != nullptr) {
    if (nrep % 4 == 0) e = sllm_launch(attn_decode_split_kernel<HD, 4, true, false>, grid, dim3(AD_WARPS * 32), 0, stream, a);
    else if (nrep % 2 == 0) e = sllm_launch(attn_decode_split_kernel<HD, 2, true, false>, grid, dim3(AD_WARPS * 32), 0, stream, a);
    else if (!a.late && (long long)a.n_split * a.G * B <= 7LL * sllm_sm_count())       // all resident at once
      e = sllm_launch(attn_decode_split_kernel<HD, 1, true, true>, grid, dim3(AD_WARPS * 32), 0, stream, a);
    else e = sllm_launch(attn_decode_split_kernel<HD, 1, true, false>, grid, dim3(AD_WARPS * 32), 0, stream, a);
  } else {
    if (nrep % 4 == 0) e = sllm_launch(attn_decode_split_kernel<HD, 4, false, false>, grid, dim3(AD_WARPS * 32), 0, stream, a);
    else if (nrep % 2 == 0) e = sllm_launch(attn_decode_split_kernel<HD, 2, false, false>, grid, dim3(AD_WARPS * 32), 0, stream, a);
    else e = sllm_launch(attn_decode_split_kernel<HD, 1, false, false>, grid, dim3(AD_WARPS * 32), 0, stream, a);
  }
  if (e != cudaSuccess || a.tickets != nullptr) return (int)e;
  return (int)sllm_launch(attn_decode_merge_kernel, dim3(a.H, B), dim3(HD < 32 ? 32 : HD), 0, stream,
                          (const float*)a.part, out, a.H, HD, a.n_split);
}

// Bytes of scratch `part` must have: B * H * n_split * (hd + 2) floats.
SLLM_EXPORT long long sllm_attn_decode_scratch_bytes(int B, int H, int hd, int n_split) {
  return (long long)B * H * n_split * (hd + 2) * (long long)sizeof(float);
}

static int attn_decode_dispatch(const void* q, int q_ld, void* out, const int* seq_pos0, const int* block_table,
                                int max_pages, const void* kpages, const void* vpages, void* scratch, int* tickets, int B,
                                int H, int G, int hd, int window, float scale, int n_split, cudaStream_t stream,
                                const void* cos_sin = nullptr, int rot = 0, int interleaved = 0, int write_kv = 0) {
  if (B <= 0) return 0;
  if (G < 1 || H % G != 0 || n_split < 1 || (q_ld & 7) || ((uintptr_t)q & 15)) return SLLM_ERR_ARG;
  if (cos_sin != nullptr && (rot < 2 || rot > hd || (rot % (interleaved ? 8 : 16)) != 0 || tickets == nullptr)) return SLLM_ERR_ARG;
  AttnDecodeArgs a{(const bf16*)q, q_ld, seq_pos0, block_table, max_pages, (const bf16*)kpages, (const bf16*)vpages,
                   (float*)scratch, H, G, window, n_split, scale, (bf16*)out, tickets, (const float2*)cos_sin, rot, interleaved,
                   write_kv, 0};
  static const int late = getenv("SLLM_DECODE_LATE_KEYS") != nullptr;   // for comparisons
  a.late = late;
  switch (hd) {
    case 16: return attn_decode_launch<16>(a, (bf16*)out, B, stream);
    case 32: return attn_decode_launch<32>(a, (bf16*)out, B, stream);
    case 64: return attn_decode_launch<64>(a, (bf16*)out, B, stream);
    case 128: return attn_decode_launch<128>(a, (bf16*)out, B, stream);
    case 256: return attn_decode_launch<256>(a, (bf16*)out, B, stream);
    default: return SLLM_ERR_ARG;   // other head widths go through the generic kernel
  }
}

// Split kernel + merge kernel; `scratch` may hold anything.
SLLM_EXPORT int sllm_attn_decode_bf16(const void* q, int q_ld, void* out, const int* seq_pos0, const int* block_table,
                                      int max_pages, const void* kpages, const void* vpages, void* scratch, int B, int H,
                                      int G, int hd, int window, float scale, int n_split, cudaStream_t stream) {
  return attn_decode_dispatch(q, q_ld, out, seq_pos0, block_table, max_pages, kpages, vpages, scratch, nullptr, B, H, G, hd,
                              window, scale, n_split, stream);
}

// One kernel: the last split to finish merges. `tickets` holds B*G ints that are zero before the
// first launch (the kernel leaves them zero); launches that share it must not overlap.
SLLM_EXPORT int sllm_attn_decode_merged_bf16(const void* q, int q_ld, void* out, const int* seq_pos0,
                                             const int* block_table, int max_pages, const void* kpages,
                                             const void* vpages, void* scratch, int* tickets, int B, int H, int G, int hd,
                                             int window, float scale, int n_split, cudaStream_t stream) {
  if (tickets == nullptr) return SLLM_ERR_ARG;
  return attn_decode_dispatch(q, q_ld, out, seq_pos0, block_table, max_pages, kpages, vpages, scratch, tickets, B, H, G, hd,
                              window, scale, n_split, stream);
}

// Rotary positions, cache write and attention of a decode step in one kernel: `qkv` holds the
// step's unrotated rows [q heads | k heads | v heads]; the queries are rotated on the fly, and with
// write_kv the new key (rotated) and value are stored at position seq_pos0[b] by the block whose key
// range holds that position. Rotary width in multiples of 16 (half pairing) or 8 (interleaved).
SLLM_EXPORT int sllm_attn_decode_rope_bf16(const void* qkv, int ld, void* out, const int* seq_pos0, const int* block_table,
                                           int max_pages, void* kpages, void* vpages, void* scratch, int* tickets,
                                           const void* cos_sin, int rot, int interleaved, int write_kv, int B, int H, int G,
                                           int hd, int window, float scale, int n_split, cudaStream_t stream) {
  if (tickets == nullptr || cos_sin == nullptr) return SLLM_ERR_ARG;
  return attn_decode_dispatch(qkv, ld, out, seq_pos0, block_table, max_pages, kpages, vpages, scratch, tickets, B, H, G, hd,
                              window, scale, n_split, stream, cos_sin, rot, interleaved, write_kv);
}

// ------------------------------------------------------------------ decode attention without any allocation
// Declared in attn_decode_noalloc.h. The split-key attention above needs scratch for its partial
// results, which its caller allocates. Some callers cannot allocate device memory at all: code
// running inside a region where the allocator must not be entered (another library's callback, a
// real-time loop that forbids cudaMalloc's implicit synchronisation, a host program that has handed
// all device memory to its own arena). For them the scratch lives in this file, in a fixed array
// that every GPU loading the library holds until the process exits.
#include "attn_decode_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[SLLM_NOALLOC_SCRATCH_FLOATS];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not an address a kernel may
// use; the device address is asked for once per device, with that device current.
#define SLLM_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[SLLM_NOALLOC_MAX_DEVICES];

SLLM_EXPORT const char* sllm_attn_decode_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case SLLM_NOALLOC_ERR_TOO_LARGE:
      return "attn_decode_noalloc: B * H * n_split * (head_dim + 2) floats exceed the built-in scratch "
             "(SLLM_NOALLOC_SCRATCH_FLOATS); use fewer splits or the entry point that takes caller scratch";
    case SLLM_NOALLOC_ERR_DEVICE: return "attn_decode_noalloc: the current device's ordinal is beyond the table of 64 devices";
    case SLLM_ERR_ARG:
      return "attn_decode_noalloc: bad arguments (head counts, a head width other than 16, 32, 64, 128 or 256, "
             "alignment of q, or n_split < 1)";
    default: return code > 0 ? "attn_decode_noalloc: CUDA error (see cudaError_t)" : "attn_decode_noalloc: unknown error code";
  }
}

SLLM_EXPORT long long sllm_attn_decode_noalloc_capacity_floats(void) { return (long long)SLLM_NOALLOC_SCRATCH_FLOATS; }

SLLM_EXPORT int sllm_attn_decode_bf16_noalloc(const void* q, int q_ld, void* out, const int* seq_pos0,
                                              const int* block_table, int max_pages, const void* kpages,
                                              const void* vpages, int B, int H, int G, int hd, int window, float scale,
                                              int n_split, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (G < 1 || H % G != 0 || n_split < 1 || hd < 1) return SLLM_ERR_ARG;
  long long need = (long long)B * H * n_split * (hd + 2);
  if (need > (long long)SLLM_NOALLOC_SCRATCH_FLOATS) return SLLM_NOALLOC_ERR_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= SLLM_NOALLOC_MAX_DEVICES) return SLLM_NOALLOC_ERR_DEVICE;
  if (g_noalloc_ptr[dev] == nullptr) {           // first call on this device: set-up (do it before any stream capture)
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = ptr;
  }
  // Nothing in the scratch has to start at zero: every block of the split kernel writes all of its
  // (sequence, head, split) entries, empty splits included, before the merge kernel reads them.
  return sllm_attn_decode_bf16(q, q_ld, out, seq_pos0, block_table, max_pages, kpages, vpages, g_noalloc_ptr[dev], B, H,
                               G, hd, window, scale, n_split, stream);
}

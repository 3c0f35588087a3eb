// Generic kernels, templated on the activation/weight element type (float or bfloat16).
//
// These are the whole kernel set of the true 32-bit path (FP32 FMA only, no tensor cores, no
// reduced-precision matrix mode) and the fall-back shapes of the bfloat16 path. Every
// accumulation, the softmax, the norms and the rotation are computed in float; only loads and
// stores see the element type.
//
// The mathematics is that of the reference's CPU functions: rmsNormFlatF32
// (float32_ops.go:159-172), applyRopeInPlaceF32 (:174-188), fusedAttentionHeadF32 (:190-235),
// the dense matmul (:462-482) and the SiLU gate (model_f32.go:484-490).
#pragma once
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :] widened to float (the residual stream is float in both paths).
// An id outside the table writes zeros and raises *err (the host checks ids before it launches).
template <typename W>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const W* __restrict__ table,
                                  float* __restrict__ out, int d, int vocab, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  int id = ids[t];
  bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0) atomicExch(err, 1);
  const W* src = table + (size_t)(ok ? id : 0) * d;
  float* dst = out + (size_t)t * d;
  for (int j = threadIdx.x; j < d; j += blockDim.x) dst[j] = ok ? to_f32(src[j]) : 0.f;
}

// ------------------------------------------------------------------ residual add + RMSNorm
// v = x[row] + delta[row]; y = (v * 1/sqrt(mean(v^2) + eps)) * w.
// delta is either one array of the element type (n_parts == 0) or n_parts float arrays
// `part_stride` elements apart whose sum is the addend (the partial sums of a product whose K
// range was split over blocks); they are added in a fixed order.
// rows == nullptr: row r of y comes from row r of x, and x is updated in place (the residual sum).
// rows != nullptr: row r of y comes from row rows[r]; x is left alone.
template <typename A, int U>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int n_parts,
                                   size_t part_stride, const int* __restrict__ rows, const void* __restrict__ w,
                                   int w_f32, A* __restrict__ y, int d, float eps) {
  extern __shared__ float sm_row[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  int r = blockIdx.x;
  size_t in = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + in * d;
  const A* dr = (delta && n_parts == 0) ? (const A*)delta + in * d : nullptr;
  const float* pr = (delta && n_parts > 0) ? (const float*)delta + in * d : nullptr;
  float ss = 0.f;
  A* yr = y + (size_t)r * d;
  bool update = (rows == nullptr) && (delta != nullptr);
  if ((d & 3) == 0) {
    // four elements per thread and access (16 bytes of the float rows), U accesses in flight before
    // the first is used: with many rows the blocks are small and each thread walks further
    for (int j0 = threadIdx.x * 4; j0 < d; j0 += blockDim.x * 4 * U) {
      float4 v[U], a[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        int j = j0 + u * blockDim.x * 4;
        v[u] = j < d ? *(const float4*)(xr + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (dr) {
#pragma unroll
        for (int u = 0; u < U; u++) {
          int j = j0 + u * blockDim.x * 4;
          a[u] = j < d ? ld_dep4(dr + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; u++) a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (pr) {
        for (int p = 0; p < n_parts; p++) {
#pragma unroll
          for (int u = 0; u < U; u++) {
            int j = j0 + u * blockDim.x * 4;
            if (j < d) {
              float4 b = ld_dep4(pr + (size_t)p * part_stride + j);
              a[u].x += b.x; a[u].y += b.y; a[u].z += b.z; a[u].w += b.w;
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        int j = j0 + u * blockDim.x * 4;
        if (j < d) {
          float4 t = make_float4(v[u].x + a[u].x, v[u].y + a[u].y, v[u].z + a[u].z, v[u].w + a[u].w);
          *(float4*)(sm_row + j) = t;
          ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        }
      }
    }
    ss = block_sum(ss, red);
    float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
      float4 v = *(const float4*)(sm_row + j);
      if (update) *(float4*)(xr + j) = v;
      float4 wv = w_f32 ? ld4((const float*)w + j) : ld4((const bf16*)w + j);
      st4(yr + j, make_float4((v.x * inv) * wv.x, (v.y * inv) * wv.y, (v.z * inv) * wv.z, (v.w * inv) * wv.w));
    }
    return;
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float v = xr[j];
    if (dr) v += to_f32(ld_dep(dr + j));
    if (pr) {
      float a = 0.f;
      for (int p = 0; p < n_parts; p++) a += ld_dep(pr + (size_t)p * part_stride + j);
      v += a;
    }
    sm_row[j] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)d + eps);
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float v = sm_row[j];
    if (update) xr[j] = v;
    yr[j] = from_f32<A>((v * inv) * load_w(w, w_f32, j));
  }
}

// ------------------------------------------------------------------ C = A * B^T, tiled, FP32 FMA
// A [M,K] (row stride lda), B [N,K] (row stride ldb: weights are [out, in]), C [M,N].
// Each output is one ascending-k chain of fused multiply-adds in float.
template <typename TI, typename TO, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_nt_tiled_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TO* __restrict__ C, int M, int N, int K,
                     int lda, int ldb, int ldc) {
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int PAD = 4;
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];
  int tid = threadIdx.x;
  int tx = tid % (BN / TN), ty = tid / (BN / TN);
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += NT) {
      int row = e / BK, kk = e % BK;
      int gm = m0 + row, gk = k0 + kk;
      As[kk][row] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
    }
    for (int e = tid; e < BN * BK; e += NT) {
      int row = e / BK, kk = e % BK;
      int gn = n0 + row, gk = k0 + kk;
      Bs[kk][row] = (gn < N && gk < K) ? to_f32(B[(size_t)gn * ldb + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; j++) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; i++) {
    int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int gn = n0 + tx * TN + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = from_f32<TO>(acc[i][j]);
    }
  }
}

// Few rows (M <= MT): every weight row is read once and used for all M rows. One warp per output
// column; lanes stride over k; warp-shuffle sum.
template <typename TI, typename TO, int MT>
__global__ void gemv_nt_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TO* __restrict__ C, int M, int N,
                               int K, int lda, int ldb, int ldc) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const TI* brow = B + (size_t)n * ldb;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  for (int k = lane; k < K; k += 32) {
    float b = to_f32(brow[k]);
#pragma unroll
    for (int m = 0; m < MT; m++)
      if (m < M) acc[m] = fmaf(to_f32(A[(size_t)m * lda + k]), b, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < MT; m++) {
    float v = warp_sum(acc[m]);
    if (lane == 0 && m < M) C[(size_t)m * ldc + n] = from_f32<TO>(v);
  }
}

// ------------------------------------------------------------------ rotary positions + cache write
// qkv row t holds [q heads | k heads | v heads], head width hd. Q and K pairs of the first `rot`
// dims are rotated by the angle of the token's absolute position (table built on the host in
// float64: cs[pos][i] = (cos, sin)(pos * f_i)); Q is rewritten in place, rotated K and raw V go
// to the token's place in the paged cache. n_kv == 0: only Q is rotated (a layer that reads
// another layer's cache).
template <typename A>
__global__ void rope_kv_write_kernel(A* __restrict__ qkv, int ld, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                     int max_pages, const float2* __restrict__ cs, A* __restrict__ kpages,
                                     A* __restrict__ vpages, int H, int n_kv, int hd, int rot, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  int pos = tok_pos[t];
  int half = rot >> 1;
  A* row = qkv + (size_t)t * ld;
  size_t cache_base = 0;
  if (n_kv > 0) {
    int page = block_table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE];
    cache_base = ((size_t)page * n_kv * SLLM_PAGE + (pos % SLLM_PAGE)) * hd;   // + g * PAGE * hd + dim
  }
  const float2* csr = cs + (size_t)pos * half;
  int n_rot = (H + n_kv) * half;
  for (int idx = threadIdx.x; idx < n_rot; idx += blockDim.x) {
    int head = idx / half, i = idx % half;
    int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    A* h = row + (size_t)head * hd;
    float x0 = to_f32(h[i0]), x1 = to_f32(h[i1]);
    float2 c = csr[i];
    float r0 = x0 * c.x - x1 * c.y;
    float r1 = x0 * c.y + x1 * c.x;
    if (head < H) {
      h[i0] = from_f32<A>(r0);
      h[i1] = from_f32<A>(r1);
    } else {
      A* dst = kpages + cache_base + (size_t)(head - H) * SLLM_PAGE * hd;
      dst[i0] = from_f32<A>(r0);
      dst[i1] = from_f32<A>(r1);
    }
  }
  if (n_kv == 0) return;
  int tail = hd - rot;
  for (int idx = threadIdx.x; idx < n_kv * tail; idx += blockDim.x) {
    int g = idx / tail, j = rot + idx % tail;
    kpages[cache_base + (size_t)g * SLLM_PAGE * hd + j] = row[(size_t)(H + g) * hd + j];
  }
  for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
    int g = idx / hd, j = idx % hd;
    vpages[cache_base + (size_t)g * SLLM_PAGE * hd + j] = row[(size_t)(H + n_kv + g) * hd + j];
  }
}

// The same with 16-byte accesses, eight elements per thread and step. Needs head width and row
// stride in multiples of 8 and a rotary width in multiples of 16 (half pairing) or 8 (interleaved).
template <typename A>
__global__ void rope_kv_write_vec_kernel(A* __restrict__ qkv, int ld, const int* __restrict__ tok_pos,
                                         const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                         int max_pages, const float2* __restrict__ cs, A* __restrict__ kpages,
                                         A* __restrict__ vpages, int H, int n_kv, int hd, int rot, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  int pos = tok_pos[t];
  int half = rot >> 1;
  A* row = qkv + (size_t)t * ld;
  size_t cache_base = 0;
  if (n_kv > 0) {
    int page = block_table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE];
    cache_base = ((size_t)page * n_kv * SLLM_PAGE + (pos % SLLM_PAGE)) * hd;
  }
  const float2* csr = cs + (size_t)pos * half;
  if (interleaved) {
    int vecs = rot >> 3;                       // 8 elements = 4 adjacent pairs
    for (int idx = threadIdx.x; idx < (H + n_kv) * vecs; idx += blockDim.x) {
      int head = idx / vecs, v = idx % vecs;
      A* h = row + (size_t)head * hd + v * 8;
      F8 x = ld8(h), y;
      const float4* c4 = (const float4*)(csr + v * 4);   // (cos, sin) of 4 pairs
#pragma unroll
      for (int i = 0; i < 2; i++) {
        float4 c = c4[i];
        y.f[4 * i] = x.f[4 * i] * c.x - x.f[4 * i + 1] * c.y;
        y.f[4 * i + 1] = x.f[4 * i] * c.y + x.f[4 * i + 1] * c.x;
        y.f[4 * i + 2] = x.f[4 * i + 2] * c.z - x.f[4 * i + 3] * c.w;
        y.f[4 * i + 3] = x.f[4 * i + 2] * c.w + x.f[4 * i + 3] * c.z;
      }
      if (head < H) st8(h, y);
      else st8(kpages + cache_base + (size_t)(head - H) * SLLM_PAGE * hd + v * 8, y);
    }
  } else {
    int vecs = half >> 3;                      // 8 first-half elements and their 8 partners
    for (int idx = threadIdx.x; idx < (H + n_kv) * vecs; idx += blockDim.x) {
      int head = idx / vecs, v = idx % vecs;
      A* h = row + (size_t)head * hd + v * 8;
      F8 x0 = ld8(h), x1 = ld8(h + half), y0, y1;
      const float4* c4 = (const float4*)(csr + v * 8);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        float4 c = c4[i];
        y0.f[2 * i] = x0.f[2 * i] * c.x - x1.f[2 * i] * c.y;
        y1.f[2 * i] = x0.f[2 * i] * c.y + x1.f[2 * i] * c.x;
        y0.f[2 * i + 1] = x0.f[2 * i + 1] * c.z - x1.f[2 * i + 1] * c.w;
        y1.f[2 * i + 1] = x0.f[2 * i + 1] * c.w + x1.f[2 * i + 1] * c.z;
      }
      if (head < H) { st8(h, y0); st8(h + half, y1); }
      else {
        A* dst = kpages + cache_base + (size_t)(head - H) * SLLM_PAGE * hd + v * 8;
        st8(dst, y0);
        st8(dst + half, y1);
      }
    }
  }
  if (n_kv == 0) return;
  int tail = (hd - rot) >> 3;
  for (int idx = threadIdx.x; idx < n_kv * tail; idx += blockDim.x) {
    int g = idx / tail, j = rot + (idx % tail) * 8;
    st8(kpages + cache_base + (size_t)g * SLLM_PAGE * hd + j, ld8(row + (size_t)(H + g) * hd + j));
  }
  int vv = hd >> 3;
  for (int idx = threadIdx.x; idx < n_kv * vv; idx += blockDim.x) {
    int g = idx / vv, j = (idx % vv) * 8;
    st8(vpages + cache_base + (size_t)g * SLLM_PAGE * hd + j, ld8(row + (size_t)(H + n_kv + g) * hd + j));
  }
}

// ------------------------------------------------------------------ attention over the paged cache
// One block: ATT_BQ consecutive queries of one sequence, one query head. Keys and values come
// from the cache (this step's own keys were written before). Key j is seen by the query at
// absolute position p when j <= p and (window == 0 or j > p - window). Online softmax in float:
// running maximum m, running sum l, accumulator rescaled when m grows.
#define ATT_BQ 16
#define ATT_BK 32
#define ATT_THREADS 128

struct AttnArgs {
  const void* q;        // [T, q_ld] rotated queries; head h at columns h*hd
  int q_ld;
  void* out;            // [T, H*hd]
  const int* seq_start; // [B+1] first row of each sequence in the packed batch
  const int* seq_pos0;  // [B] cache length of each sequence before this step
  const int* block_table;
  int max_pages;
  const void* kpages;   // [pages][G][PAGE][hd]
  const void* vpages;
  int H, G, hd, window;
  float scale;
};

template <typename A, int NACC>
__global__ void __launch_bounds__(ATT_THREADS) attn_paged_kernel(AttnArgs p) {
  extern __shared__ float att_sm[];
  const int hd = p.hd;
  float* Qs = att_sm;                          // [ATT_BQ][hd]
  float* Ks = Qs + ATT_BQ * hd;                // [ATT_BK][hd + 1]
  float* Vs = Ks + ATT_BK * (hd + 1);          // [ATT_BK][hd]
  int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  int row0 = p.seq_start[b], S = p.seq_start[b + 1] - row0;
  int r0 = qt * ATT_BQ;
  if (r0 >= S) return;
  int nq = min(ATT_BQ, S - r0);
  int pos0 = p.seq_pos0[b];
  int g = h / (p.H / p.G);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const A* q = (const A*)p.q;
  const A* kp = (const A*)p.kpages;
  const A* vp = (const A*)p.vpages;

  for (int e = threadIdx.x; e < ATT_BQ * hd; e += ATT_THREADS) {
    int qi = e / hd, dd = e % hd;
    Qs[e] = (qi < nq) ? to_f32(q[(size_t)(row0 + r0 + qi) * p.q_ld + (size_t)h * hd + dd]) : 0.f;
  }

  constexpr int QPW = ATT_BQ / (ATT_THREADS / 32);   // queries per warp
  float m[QPW], l[QPW], acc[QPW][NACC];
#pragma unroll
  for (int i = 0; i < QPW; i++) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int a = 0; a < NACC; a++) acc[i][a] = 0.f;
  }

  int k_hi = pos0 + r0 + nq;                                   // one past the last key any query sees
  int k_lo = p.window > 0 ? max(0, pos0 + r0 - p.window + 1) : 0;
  k_lo = (k_lo / ATT_BK) * ATT_BK;
  const int* bt = p.block_table + (size_t)b * p.max_pages;

  for (int kt = k_lo; kt < k_hi; kt += ATT_BK) {
    int page = bt[kt / SLLM_PAGE];
    size_t base = ((size_t)page * p.G + g) * SLLM_PAGE * hd + (size_t)(kt % SLLM_PAGE) * hd;
    __syncthreads();
    for (int e = threadIdx.x; e < ATT_BK * hd; e += ATT_THREADS) {
      int kk = e / hd, dd = e % hd;
      bool ok = page >= 0 && (kt + kk) < k_hi;
      Ks[kk * (hd + 1) + dd] = ok ? to_f32(kp[base + e]) : 0.f;
      Vs[e] = ok ? to_f32(vp[base + e]) : 0.f;
    }
    __syncthreads();
    int kpos = kt + lane;
#pragma unroll
    for (int i = 0; i < QPW; i++) {
      int qi = warp * QPW + i;
      if (qi >= nq) continue;                                  // uniform per warp
      int qpos = pos0 + r0 + qi;
      const float* qv = Qs + qi * hd;
      const float* kv = Ks + lane * (hd + 1);
      float dot = 0.f;
      for (int dd = 0; dd < hd; dd++) dot = fmaf(qv[dd], kv[dd], dot);
      float s = dot * p.scale;
      bool seen = page >= 0 && kpos <= qpos && (p.window == 0 || kpos > qpos - p.window);
      if (!seen) s = -INFINITY;
      float m_new = fmaxf(m[i], warp_max(s));
      if (m_new == -INFINITY) continue;                        // nothing seen yet by this query
      float pr = seen ? expf(s - m_new) : 0.f;
      float corr = expf(m[i] - m_new);                         // exp(-inf) = 0 on the first tile
      l[i] = l[i] * corr + warp_sum(pr);
      m[i] = m_new;
#pragma unroll
      for (int a = 0; a < NACC; a++) acc[i][a] *= corr;
      for (int kk = 0; kk < ATT_BK; kk++) {
        float pk = __shfl_sync(0xffffffffu, pr, kk);
#pragma unroll
        for (int a = 0; a < NACC; a++) {
          int dd = lane + 32 * a;
          if (dd < hd) acc[i][a] = fmaf(pk, Vs[kk * hd + dd], acc[i][a]);
        }
      }
    }
  }
  A* out = (A*)p.out;
#pragma unroll
  for (int i = 0; i < QPW; i++) {
    int qi = warp * QPW + i;
    if (qi >= nq) continue;
    float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
    for (int a = 0; a < NACC; a++) {
      int dd = lane + 32 * a;
      if (dd < hd) out[(size_t)(row0 + r0 + qi) * ((size_t)p.H * hd) + (size_t)h * hd + dd] = from_f32<A>(acc[i][a] * inv);
    }
  }
}

// ------------------------------------------------------------------ SiLU-gated product
// gu [T, 2F]. tiled == 0: gate in columns [0,F), up in [F,2F). tiled != 0: columns come in tiles
// of 16, 8 gate columns then the 8 matching up columns (the row order the stacked weight is kept
// in, so that a tensor-core tile holds both halves of a pair).
// h = g * (1/(1+exp(-g))) * u, left to right.
template <typename A>
__global__ void swiglu_kernel(const A* __restrict__ gu, A* __restrict__ h, int F, size_t n, int tiled) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  size_t t = i / F;
  int j = (int)(i % F);
  int gc = tiled ? (j >> 3) * 16 + (j & 7) : j;
  int uc = tiled ? gc + 8 : F + j;
  float g = to_f32(gu[t * 2 * F + gc]);
  float u = to_f32(gu[t * 2 * F + uc]);
  float s = 1.0f / (1.0f + expf(-g));
  h[i] = from_f32<A>(g * s * u);
}

// widen / narrow a buffer (a matrix kept in 32-bit inside a bfloat16 model runs in 32-bit)
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f32<TO>(to_f32(in[i]));
}

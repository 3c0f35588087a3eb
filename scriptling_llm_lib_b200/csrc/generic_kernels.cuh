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

// The same product for many rows with register tiles: a block of 256 threads owns a BM x 128 tile of
// C, a thread (BM/16) x 8 outputs as (BM/64) x 2 groups of 4 x 4, 64 columns / rows apart so that its
// operands are 16-byte shared-memory loads. A and B tiles of 16 k are fetched from global memory as
// 16-byte vectors into registers while the previous tile is multiplied, then stored k-major
// (transposed) into the other of two shared buffers: one barrier per tile. Each output is still one
// ascending-k chain of fused multiply-adds in float. Needs K, lda, ldb in multiples of 4 elements
// and 16-byte (float) / 8-byte (bfloat16) aligned rows; the launcher falls back to the kernel above
// otherwise. With several blocks along blockIdx.z, block z takes the z-th contiguous part of K
// (k_per_split elements, a multiple of 16) and C receives float partial sums at C + z * M * ldc.
template <typename TI, typename TO, int BM>
__global__ void __launch_bounds__(256, 2)
gemm_nt_regtile_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TO* __restrict__ C, int M, int N, int K,
                       int lda, int ldb, int ldc, int k_per_split) {
  constexpr int BN = 128, BK = 16, TMG = BM / 64;          // TMG groups of 4 rows per thread
  constexpr int A_VEC = BM * BK / 4 / 256;                 // 16-byte vectors of the A tile per thread (1 or 2)
  constexpr int B_VEC = BN * BK / 4 / 256;                 // 2
  __shared__ __align__(16) float As[2][BK][BM];
  __shared__ __align__(16) float Bs[2][BK][BN];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int k_begin = blockIdx.z * k_per_split, k_end = min(K, k_begin + k_per_split);
  TO* Cz = C + (size_t)blockIdx.z * M * ldc;

  float acc[TMG * 4][8];
#pragma unroll
  for (int i = 0; i < TMG * 4; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

  // vector v of this thread: row = (tid + 256 v) % rows, k quad = (tid + 256 v) / rows: a warp reads 32
  // consecutive rows at one k quad, and stores 32 consecutive floats of one k row (no bank conflict)
  float4 ra[A_VEC], rb[B_VEC];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int v = 0; v < A_VEC; v++) {
      int e = tid + 256 * v, row = e % BM, kq = e / BM;
      int gm = m0 + row, gk = k0 + kq * 4;
      ra[v] = (gm < M && gk < k_end) ? ld4(A + (size_t)gm * lda + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int v = 0; v < B_VEC; v++) {
      int e = tid + 256 * v, row = e % BN, kq = e / BN;
      int gn = n0 + row, gk = k0 + kq * 4;
      rb[v] = (gn < N && gk < k_end) ? ld4(B + (size_t)gn * ldb + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int v = 0; v < A_VEC; v++) {
      int e = tid + 256 * v, row = e % BM, kq = e / BM;
      As[buf][kq * 4 + 0][row] = ra[v].x; As[buf][kq * 4 + 1][row] = ra[v].y;
      As[buf][kq * 4 + 2][row] = ra[v].z; As[buf][kq * 4 + 3][row] = ra[v].w;
    }
#pragma unroll
    for (int v = 0; v < B_VEC; v++) {
      int e = tid + 256 * v, row = e % BN, kq = e / BN;
      Bs[buf][kq * 4 + 0][row] = rb[v].x; Bs[buf][kq * 4 + 1][row] = rb[v].y;
      Bs[buf][kq * 4 + 2][row] = rb[v].z; Bs[buf][kq * 4 + 3][row] = rb[v].w;
    }
  };

  fetch(k_begin);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = k_begin; k0 < k_end; k0 += BK) {
    const bool more = k0 + BK < k_end;
    if (more) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TMG * 4], b[8];
#pragma unroll
      for (int g = 0; g < TMG; g++) {
        float4 t = *(const float4*)&As[buf][kk][g * 64 + ty * 4];
        a[4 * g] = t.x; a[4 * g + 1] = t.y; a[4 * g + 2] = t.z; a[4 * g + 3] = t.w;
      }
#pragma unroll
      for (int g = 0; g < 2; g++) {
        float4 t = *(const float4*)&Bs[buf][kk][g * 64 + tx * 4];
        b[4 * g] = t.x; b[4 * g + 1] = t.y; b[4 * g + 2] = t.z; b[4 * g + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TMG * 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
  const bool vec_out = (ldc & 3) == 0 && ((uintptr_t)Cz % (4 * sizeof(TO))) == 0;
#pragma unroll
  for (int i = 0; i < TMG * 4; i++) {
    int gm = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (gm >= M) continue;
#pragma unroll
    for (int g = 0; g < 2; g++) {
      int gn = n0 + g * 64 + tx * 4;
      TO* dst = Cz + (size_t)gm * ldc + gn;
      if (vec_out && gn + 3 < N) {
        st4(dst, make_float4(acc[i][4 * g], acc[i][4 * g + 1], acc[i][4 * g + 2], acc[i][4 * g + 3]));
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (gn + j < N) dst[j] = from_f32<TO>(acc[i][4 * g + j]);
      }
    }
  }
}

// Few rows (M <= MT): every weight row is read from memory once and used for all M rows. A block of
// 256 threads owns NC output columns; its threads split K in 16-byte vectors (thread t takes elements
// 4t.., 4(t+256)..), so the block streams NC weight rows with every load of the warp contiguous; the
// M x NC partial sums of a thread are folded across the warp by a reduce-scatter (31 shuffles for 32
// sums) and across the warps through shared memory in a fixed order. With KSPLIT blocks along
// blockIdx.y, block y takes the y-th contiguous part of K and C receives float partial sums at
// C + y * M * ldc (the reader, a norm, adds them). Needs K, lda, ldb in multiples of 4 elements.
template <typename TI, typename TO, int MT, int NC>
__global__ void __launch_bounds__(256, 2)
gemv_nt_block_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TO* __restrict__ C, int M, int N, int K,
                     int lda, int ldb, int ldc, int k_per_split) {
  constexpr int NV = MT * NC;                              // sums per thread; a power of two, 4..64
  __shared__ float red[8][NV];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * NC;
  const int k_begin = blockIdx.y * k_per_split, k_end = min(K, k_begin + k_per_split);
  TO* Cz = C + (size_t)blockIdx.y * M * ldc;
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) acc[i] = 0.f;
  const TI* brow[NC];
#pragma unroll
  for (int c = 0; c < NC; c++) brow[c] = B + (size_t)min(n0 + c, N - 1) * ldb;

  for (int k = k_begin + tid * 4; k < k_end; k += 256 * 4) {
    float4 b[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) b[c] = ld4_stream(brow[c] + k);
#pragma unroll
    for (int m = 0; m < MT; m++) {
      float4 a = (m < M) ? ld4(A + (size_t)m * lda + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < NC; c++) {
        float s = acc[m * NC + c];
        s = fmaf(a.x, b[c].x, s); s = fmaf(a.y, b[c].y, s); s = fmaf(a.z, b[c].z, s); s = fmaf(a.w, b[c].w, s);
        acc[m * NC + c] = s;
      }
    }
  }
  // reduce-scatter over the warp: after the step with offset o a lane keeps the half of its sums that
  // its bit o selects (a contiguous range of the original indices, starting at `held`); five steps
  // leave NV / 32 sums per lane (one, or two when a thread had 64), fewer steps leave one that the
  // lanes sharing it still have to add up
  int held = 0;
  constexpr int STEPS = NV >= 32 ? 5 : (NV == 16 ? 4 : (NV == 8 ? 3 : 2));
  constexpr int LEFT = NV >> STEPS;                            // sums per lane afterwards: 1 or 2
#pragma unroll
  for (int st = 0; st < STEPS; st++) {
    const int n = NV >> st, o = 16 >> st;
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; i++) {
      float keep = up ? acc[i + n / 2] : acc[i];
      float send = up ? acc[i] : acc[i + n / 2];
      acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
    if (up) held += n / 2;
  }
#pragma unroll
  for (int o = 16 >> STEPS; o > 0; o >>= 1)                    // lanes that hold the same index (fewer than 32 sums)
#pragma unroll
    for (int i = 0; i < LEFT; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if ((lane & ((32 >> STEPS) - 1)) == 0) {
#pragma unroll
    for (int i = 0; i < LEFT; i++) red[warp][held + i] = acc[i];
  }
  __syncthreads();
  if (tid < NV) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) t += red[w][tid];
    int m = tid / NC, c = tid % NC;
    if (m < M && n0 + c < N) Cz[(size_t)m * ldc + n0 + c] = from_f32<TO>(t);
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

// ------------------------------------------------------------------ the same attention with register tiles
// One block of 256 threads: 64 consecutive queries of one sequence and one query head against tiles of
// 64 keys. Thread (ty = tid / 16, tx = tid % 16) owns queries 4ty..4ty+3; of the scores it owns keys
// 4tx..4tx+3 of the tile, of the output the dims 4(tx + 16g)..+3. Scores S = Q K^T and the output
// O += P V are small FMA products out of shared memory with 16-byte loads: Q and the key tile are
// kept k-major (transposed: Qs[d][query], Ks[d][key]), the values row-major, the probabilities
// row-major with a padded stride. Softmax statistics live in registers, the row maximum and sum are
// folded over the 16 lanes that share a query. The same mathematics and masks as the kernel above;
// head widths in multiples of 4 up to 64 * NG.
#define ATT2_BQ 64
#define ATT2_BK 64
#define ATT2_PS (ATT2_BK + 4)

template <typename A, int NG>
__global__ void __launch_bounds__(256) attn_paged_tiled_kernel(AttnArgs p) {
  extern __shared__ __align__(16) float att_sm[];
  const int hd = p.hd;
  float* Qs = att_sm;                          // [hd][64]
  float* Ks = Qs + hd * ATT2_BQ;               // [hd][64]
  float* Vs = Ks + hd * ATT2_BK;               // [64][hd]
  float* Ps = Vs + ATT2_BK * hd;               // [64][68]
  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int row0 = p.seq_start[b], S = p.seq_start[b + 1] - row0;
  const int r0 = qt * ATT2_BQ;
  if (r0 >= S) return;
  const int nq = min(ATT2_BQ, S - r0);
  const int pos0 = p.seq_pos0[b];
  const int g = h / (p.H / p.G);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const A* q = (const A*)p.q;
  const A* kp = (const A*)p.kpages;
  const A* vp = (const A*)p.vpages;
  const int vec_per_row = hd >> 2;

  for (int e = tid; e < ATT2_BQ * vec_per_row; e += 256) {
    int qi = e % ATT2_BQ, dq = e / ATT2_BQ;
    float4 v = qi < nq ? ld4(q + (size_t)(row0 + r0 + qi) * p.q_ld + (size_t)h * hd + dq * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    Qs[(dq * 4 + 0) * ATT2_BQ + qi] = v.x; Qs[(dq * 4 + 1) * ATT2_BQ + qi] = v.y;
    Qs[(dq * 4 + 2) * ATT2_BQ + qi] = v.z; Qs[(dq * 4 + 3) * ATT2_BQ + qi] = v.w;
  }

  float m[4], l[4], o[4][NG][4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int gg = 0; gg < NG; gg++)
#pragma unroll
      for (int c = 0; c < 4; c++) o[i][gg][c] = 0.f;
  }
  const int k_hi = pos0 + r0 + nq;
  int k_lo = p.window > 0 ? max(0, pos0 + r0 - p.window + 1) : 0;
  k_lo = (k_lo / ATT2_BK) * ATT2_BK;
  const int* bt = p.block_table + (size_t)b * p.max_pages;

  for (int kt = k_lo; kt < k_hi; kt += ATT2_BK) {
    const int page = bt[kt / SLLM_PAGE];               // a tile is one page (both are 64 keys)
    const size_t base = ((size_t)max(page, 0) * p.G + g) * SLLM_PAGE * hd;
    __syncthreads();
    for (int e = tid; e < ATT2_BK * vec_per_row; e += 256) {
      int kk = e % ATT2_BK, dq = e / ATT2_BK;
      bool ok = page >= 0 && kt + kk < k_hi;
      float4 v = ok ? ld4(kp + base + (size_t)kk * hd + dq * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      Ks[(dq * 4 + 0) * ATT2_BK + kk] = v.x; Ks[(dq * 4 + 1) * ATT2_BK + kk] = v.y;
      Ks[(dq * 4 + 2) * ATT2_BK + kk] = v.z; Ks[(dq * 4 + 3) * ATT2_BK + kk] = v.w;
    }
    for (int e = tid; e < ATT2_BK * vec_per_row; e += 256) {
      int kk = e / vec_per_row, dq = e % vec_per_row;
      bool ok = page >= 0 && kt + kk < k_hi;
      float4 v = ok ? ld4(vp + base + (size_t)kk * hd + dq * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      *(float4*)(Vs + kk * hd + dq * 4) = v;
    }
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) s[i][j] = 0.f;
#pragma unroll 4
    for (int dd = 0; dd < hd; dd++) {
      float4 qa = *(const float4*)(Qs + dd * ATT2_BQ + ty * 4);
      float4 kb = *(const float4*)(Ks + dd * ATT2_BK + tx * 4);
      const float qv[4] = {qa.x, qa.y, qa.z, qa.w}, kv[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int qi = ty * 4 + i, qpos = pos0 + r0 + qi;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int kpos = kt + tx * 4 + j;
        bool seen = page >= 0 && qi < nq && kpos <= qpos && (p.window == 0 || kpos > qpos - p.window);
        s[i][j] = seen ? s[i][j] * p.scale : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int off = 1; off < 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      float m_new = fmaxf(m[i], mx);
      float corr = (m_new == -INFINITY) ? 1.f : expf(m[i] - m_new);     // exp(-inf) = 0 on the first tile seen
      float pr[4], rs = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        pr[j] = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - m_new);
        rs += pr[j];
      }
      l[i] = l[i] * corr + rs;                                          // this lane's share of the row sum
      m[i] = m_new;
#pragma unroll
      for (int gg = 0; gg < NG; gg++)
#pragma unroll
        for (int c = 0; c < 4; c++) o[i][gg][c] *= corr;
      *(float4*)(Ps + qi * ATT2_PS + tx * 4) = make_float4(pr[0], pr[1], pr[2], pr[3]);
    }
    __syncthreads();
#pragma unroll 2
    for (int k4 = 0; k4 < ATT2_BK; k4 += 4) {
      float pv[4][4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        float4 t = *(const float4*)(Ps + (ty * 4 + i) * ATT2_PS + k4);
        pv[i][0] = t.x; pv[i][1] = t.y; pv[i][2] = t.z; pv[i][3] = t.w;
      }
#pragma unroll
      for (int gg = 0; gg < NG; gg++) {
        const int d0 = (tx + 16 * gg) * 4;
        if (d0 >= hd) continue;
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
          float4 vv = *(const float4*)(Vs + (k4 + kk) * hd + d0);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            o[i][gg][0] = fmaf(pv[i][kk], vv.x, o[i][gg][0]);
            o[i][gg][1] = fmaf(pv[i][kk], vv.y, o[i][gg][1]);
            o[i][gg][2] = fmaf(pv[i][kk], vv.z, o[i][gg][2]);
            o[i][gg][3] = fmaf(pv[i][kk], vv.w, o[i][gg][3]);
          }
        }
      }
    }
  }
  A* out = (A*)p.out;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int qi = ty * 4 + i;
    float ls = l[i];
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) ls += __shfl_xor_sync(0xffffffffu, ls, off);
    if (qi >= nq) continue;
    const float inv = ls > 0.f ? 1.0f / ls : 0.f;
#pragma unroll
    for (int gg = 0; gg < NG; gg++) {
      const int d0 = (tx + 16 * gg) * 4;
      if (d0 >= hd) continue;
      st4(out + (size_t)(row0 + r0 + qi) * ((size_t)p.H * hd) + (size_t)h * hd + d0,
          make_float4(o[i][gg][0] * inv, o[i][gg][1] * inv, o[i][gg][2] * inv, o[i][gg][3] * inv));
    }
  }
}

// ------------------------------------------------------------------ one query per sequence, keys split over blocks
// The decode step of the generic path: block (split, key/value head, sequence) streams its share of
// the sequence's pages once for up to NREP of the query heads that share the key/value head (more
// heads: once per NREP of them), LPK lanes per key with 4 dims each per pass (NV passes for wide
// heads), online softmax per lane group and head in float (exponentials as 2^x of scores scaled by
// log2 e), folded over the warp and the block. With one split the block writes the output row; otherwise it leaves
// (unnormalised sum, maximum, sum) in `part` [B][H][n_split][hd + 2] for the merge kernel below.
struct AttnSplitArgs {
  const void* q;        // [B, q_ld] rotated queries of this step
  int q_ld;
  void* out;            // [B, H*hd]
  const int* seq_pos0;  // [B] position of the query: the cache holds keys 0..pos
  const int* block_table;
  int max_pages;
  const void* kpages;
  const void* vpages;
  float* part;
  int H, G, hd, window, n_split;
  float scale;
};
#define ATT_LOG2E 1.4426950408889634f

template <typename A, int LPK, int NV, int NREP>
__global__ void __launch_bounds__(128) attn_decode_split_generic_kernel(AttnSplitArgs p) {
  constexpr int KPW = 32 / LPK;                 // keys a warp reads per load
  constexpr int UN = NV == 1 ? 4 : (NV == 2 ? 2 : 1);   // loads in flight per lane group
  extern __shared__ __align__(16) float ad_sm[];        // [4 warps][NREP][hd] partial outputs, then [4][NREP][2] (m, l)
  const int hd = p.hd;
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int nrep = p.H / p.G;                   // query heads that share this key/value head: served NREP at a time
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = lane / LPK, dl = (lane % LPK) * 4;
  const int pos = p.seq_pos0[b];
  const int k_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int pb = k_begin / SLLM_PAGE, pe = pos / SLLM_PAGE;
  const int pps = (pe - pb + p.n_split) / p.n_split;
  const int p0 = pb + split * pps, p1 = min(pe + 1, p0 + pps);
  const int k_lo = max(k_begin, p0 * SLLM_PAGE), k_hi = min(pos + 1, p1 * SLLM_PAGE);
  const int* bt = p.block_table + (size_t)b * p.max_pages;
  const A* kp = (const A*)p.kpages;
  const A* vp = (const A*)p.vpages;
  float* sm_acc = ad_sm;                        // [4][NREP][hd]
  float* sm_ml = ad_sm + 4 * NREP * hd;         // [4][NREP][2]

  for (int r0 = 0; r0 < nrep; r0 += NREP) {
    float qv[NREP][NV][4], acc[NREP][NV][4], m[NREP], l[NREP];
#pragma unroll
    for (int r = 0; r < NREP; r++) {
      const int h = g * nrep + min(r0 + r, nrep - 1);           // heads past the group's last repeat it (not stored)
      const A* qrow = (const A*)p.q + (size_t)b * p.q_ld + (size_t)h * hd;
#pragma unroll
      for (int v = 0; v < NV; v++) {
        int d = dl + v * LPK * 4;
        float4 t = d < hd ? ld4(qrow + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float sc = p.scale * ATT_LOG2E;
        qv[r][v][0] = t.x * sc; qv[r][v][1] = t.y * sc; qv[r][v][2] = t.z * sc; qv[r][v][3] = t.w * sc;
        acc[r][v][0] = acc[r][v][1] = acc[r][v][2] = acc[r][v][3] = 0.f;
      }
      m[r] = -INFINITY;
      l[r] = 0.f;
    }
    for (int kb = k_lo + warp * KPW * UN; kb < k_hi; kb += 4 * KPW * UN) {
      float4 kr[UN][NV], vr[UN][NV];
      bool ok[UN];
#pragma unroll
      for (int u = 0; u < UN; u++) {
        int key = kb + u * KPW + slot;
        ok[u] = key < k_hi;
        int kk = ok[u] ? key : k_lo;
        int page = bt[kk / SLLM_PAGE];
        size_t off = (((size_t)page * p.G + g) * SLLM_PAGE + (kk % SLLM_PAGE)) * hd;
#pragma unroll
        for (int v = 0; v < NV; v++) {
          int d = dl + v * LPK * 4;
          kr[u][v] = d < hd ? ld4(kp + off + d) : make_float4(0.f, 0.f, 0.f, 0.f);
          vr[u][v] = d < hd ? ld4(vp + off + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int r = 0; r < NREP; r++) {
        float s[UN], m_new = m[r];
#pragma unroll
        for (int u = 0; u < UN; u++) {
          float d = 0.f;
#pragma unroll
          for (int v = 0; v < NV; v++) {
            d = fmaf(qv[r][v][0], kr[u][v].x, d); d = fmaf(qv[r][v][1], kr[u][v].y, d);
            d = fmaf(qv[r][v][2], kr[u][v].z, d); d = fmaf(qv[r][v][3], kr[u][v].w, d);
          }
#pragma unroll
          for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          s[u] = ok[u] ? d : -INFINITY;
          m_new = fmaxf(m_new, s[u]);
        }
        if (m_new == -INFINITY) continue;
        float corr = exp2f(m[r] - m_new);
        m[r] = m_new;
        l[r] *= corr;
#pragma unroll
        for (int v = 0; v < NV; v++) { acc[r][v][0] *= corr; acc[r][v][1] *= corr; acc[r][v][2] *= corr; acc[r][v][3] *= corr; }
#pragma unroll
        for (int u = 0; u < UN; u++) {
          float pr = exp2f(s[u] - m_new);
          l[r] += pr;
#pragma unroll
          for (int v = 0; v < NV; v++) {
            acc[r][v][0] = fmaf(pr, vr[u][v].x, acc[r][v][0]); acc[r][v][1] = fmaf(pr, vr[u][v].y, acc[r][v][1]);
            acc[r][v][2] = fmaf(pr, vr[u][v].z, acc[r][v][2]); acc[r][v][3] = fmaf(pr, vr[u][v].w, acc[r][v][3]);
          }
        }
      }
    }
    // fold the key slots of the warp, then the warps
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
        for (int v = 0; v < NV; v++)
#pragma unroll
          for (int c = 0; c < 4; c++) {
            float ao = __shfl_xor_sync(0xffffffffu, acc[r][v][c], o);
            acc[r][v][c] = acc[r][v][c] * c1 + ao * c2;
          }
      }
      if (lane < LPK) {
#pragma unroll
        for (int v = 0; v < NV; v++) {
          int d = dl + v * LPK * 4;
          if (d < hd) *(float4*)(sm_acc + (warp * NREP + r) * hd + d) = make_float4(acc[r][v][0], acc[r][v][1], acc[r][v][2], acc[r][v][3]);
        }
        if (lane == 0) { sm_ml[(warp * NREP + r) * 2] = m[r]; sm_ml[(warp * NREP + r) * 2 + 1] = l[r]; }
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < NREP * hd; e += 128) {
      const int r = e / hd, dd = e % hd;
      if (r0 + r >= nrep) continue;
      const int h = g * nrep + r0 + r;
      float mn = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; w++) mn = fmaxf(mn, sm_ml[(w * NREP + r) * 2]);
      float a = 0.f, ls = 0.f;
#pragma unroll
      for (int w = 0; w < 4; w++) {
        float cw = mn == -INFINITY ? 0.f : exp2f(sm_ml[(w * NREP + r) * 2] - mn);
        a += sm_acc[(w * NREP + r) * hd + dd] * cw;
        ls += sm_ml[(w * NREP + r) * 2 + 1] * cw;
      }
      if (p.n_split == 1) {
        ((A*)p.out)[((size_t)b * p.H + h) * hd + dd] = from_f32<A>(ls > 0.f ? a / ls : 0.f);
      } else {
        float* dst = p.part + (((size_t)b * p.H + h) * p.n_split + split) * (hd + 2);
        dst[dd] = a;
        if (dd == 0) { dst[hd] = mn; dst[hd + 1] = ls; }
      }
    }
    __syncthreads();
  }
}

// out[b, h*hd + d] = sum_s acc_s[d] 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits added in order
template <typename A>
__global__ void attn_split_merge_kernel(const float* __restrict__ part, A* __restrict__ out, int H, int hd, int n_split) {
  const int h = blockIdx.x, b = blockIdx.y;
  const float* src = part + ((size_t)b * H + h) * n_split * (hd + 2);
  float mn = -INFINITY;
  for (int s2 = 0; s2 < n_split; s2++) mn = fmaxf(mn, src[(size_t)s2 * (hd + 2) + hd]);
  for (int dd = threadIdx.x; dd < hd; dd += blockDim.x) {
    float a = 0.f, ls = 0.f;
    for (int s2 = 0; s2 < n_split; s2++) {
      const float* ps = src + (size_t)s2 * (hd + 2);
      float c = (mn == -INFINITY || ps[hd] == -INFINITY) ? 0.f : exp2f(ps[hd] - mn);
      a += ps[dd] * c;
      ls += ps[hd + 1] * c;
    }
    out[((size_t)b * H + h) * hd + dd] = from_f32<A>(ls > 0.f ? a / ls : 0.f);
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

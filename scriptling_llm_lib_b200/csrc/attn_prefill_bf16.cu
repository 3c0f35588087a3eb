// Causal grouped-query attention of a prompt step over the paged cache, bfloat16, on tensor cores.
//
// One block: 64 consecutive queries of one sequence and one query head (16 per warp). Keys and
// values are read a page (64 positions) at a time straight from the cache -- this step's own keys
// were written there before -- with cp.async into swizzled shared memory, double buffered.
// S = Q K^T and O += P V run on mma.sync.m16n8k16 (bfloat16 in, float accumulate); the softmax is
// the online form in float (running maximum and sum per query row, accumulator rescaled when the
// maximum grows), in base 2 with the scale folded in. Same mathematics as fusedAttentionHeadF32
// (float32_ops.go:190-235): key j is seen by the query at position p when j <= p, and with a
// window only when j > p - window.
//
// Head widths 64 and 128; other widths go through the generic kernel.
#include "common.cuh"

#define FA_BQ 64
#define FA_BK 64          // = SLLM_PAGE: a key tile is one page of one key/value head
#define FA_THREADS 128
#define FA_LOG2E 1.4426950408889634f

struct FaArgs {
  const bf16* q;        // [T, q_ld], head h at columns h*HD (rotated)
  int q_ld;
  bf16* out;            // [T, H*HD]
  const int* seq_start; // [B+1]
  const int* seq_pos0;  // [B]
  const int* block_table;
  int max_pages;
  const bf16* kpages;   // [pages][G][PAGE][HD]
  const bf16* vpages;
  int H, G, window;
  float scale;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int n = valid ? 16 : 0;    // 0 bytes read: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// byte offset of the 16-byte chunk `c` of row `r` in a tile with rows of HD bfloat16, chunks
// XOR-swizzled with the row so that 8 rows read by one ldmatrix fall into 8 different bank groups
template <int HD> __device__ __forceinline__ uint32_t tile_off(int r, int c) {
  return (uint32_t)(r * (HD * 2) + ((c ^ (r & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS) attn_prefill_kernel(FaArgs p) {
  constexpr int CH = HD / 8;           // 16-byte chunks per row
  constexpr int KS = HD / 16;          // k-steps of the QK^T product
  constexpr int TILE = FA_BK * HD * 2; // bytes of one K or V tile
  extern __shared__ __align__(128) uint8_t fa_smem[];
  const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(fa_smem);
  const uint32_t sK = sQ + FA_BQ * HD * 2, sV = sK + 2 * TILE;

  // heads vary fastest, query tiles from the last (most keys) to the first: blocks start in the order
  // of their length over the whole grid, so the long ones are not left for the end
  int b = blockIdx.z, h = blockIdx.x, qt = gridDim.y - 1 - blockIdx.y;
  int row0 = p.seq_start[b], S = p.seq_start[b + 1] - row0;
  int r0 = qt * FA_BQ;
  if (r0 >= S) return;
  int nq = min(FA_BQ, S - r0);
  int pos0 = p.seq_pos0[b];
  int g = h / (p.H / p.G);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int* bt = p.block_table + (size_t)b * p.max_pages;

  int q_lo = pos0 + r0, q_hi = pos0 + r0 + nq - 1;            // positions of the tile's first and last query
  int k_first = p.window > 0 ? max(0, q_lo - p.window + 1) : 0;
  int t_lo = k_first / FA_BK, t_hi = q_hi / FA_BK;            // key tiles (pages) to visit

  // ---- Q tile -> shared (rows past the sequence are zero)
  for (int e = threadIdx.x; e < FA_BQ * CH; e += FA_THREADS) {
    int r = e / CH, c = e % CH;
    const bf16* src = p.q + (size_t)(row0 + r0 + min(r, nq - 1)) * p.q_ld + (size_t)h * HD + c * 8;
    cp_async16(sQ + tile_off<HD>(r, c), src, r < nq);
  }
  auto load_kv = [&](int t, int buf) {
    int page = bt[t];
    int n_valid = min(FA_BK, q_hi + 1 - t * FA_BK);           // keys of this page any query of the tile may see
    const bf16* kb = p.kpages + ((size_t)page * p.G + g) * (FA_BK * HD);
    const bf16* vb = p.vpages + ((size_t)page * p.G + g) * (FA_BK * HD);
    for (int e = threadIdx.x; e < FA_BK * CH; e += FA_THREADS) {
      int r = e / CH, c = e % CH;
      bool ok = page >= 0 && r < n_valid;
      size_t off = ok ? (size_t)r * HD + c * 8 : 0;
      cp_async16(sK + buf * TILE + tile_off<HD>(r, c), ok ? kb + off : p.kpages, ok);
      cp_async16(sV + buf * TILE + tile_off<HD>(r, c), ok ? vb + off : p.vpages, ok);
    }
  };
  load_kv(t_lo, 0);
  cp_async_commit();

  uint32_t qf[KS][4];
  float o[HD / 8][4], m[2], l[2];
#pragma unroll
  for (int i = 0; i < HD / 8; i++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[i][e] = 0.f;
  m[0] = m[1] = -INFINITY;
  l[0] = l[1] = 0.f;
  const float sc = p.scale * FA_LOG2E;
  int qrow = warp * 16;                                        // this warp's rows in the tile
  int qpos_a = pos0 + r0 + qrow + gid, qpos_b = qpos_a + 8;     // positions of the two rows a thread holds

  for (int t = t_lo; t <= t_hi; t++) {
    int buf = (t - t_lo) & 1;
    if (t < t_hi) load_kv(t + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (t == t_lo) {
#pragma unroll
      for (int ks = 0; ks < KS; ks++)
        ldsm_x4(sQ + tile_off<HD>(qrow + (lane & 15), ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
      for (int e = 0; e < 4; e++) s[i][e] = 0.f;
    const uint32_t kbase = sK + buf * TILE, vbase = sV + buf * TILE;
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
      for (int np = 0; np < 4; np++) {
        uint32_t b0, b1, b2, b3;
        int krow = np * 16 + ((lane >> 4) << 3) + (lane & 7);
        ldsm_x4(kbase + tile_off<HD>(krow, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma16816(s[2 * np], qf[ks], b0, b1);
        mma16816(s[2 * np + 1], qf[ks], b2, b3);
      }
    }
    // ---- mask, online softmax. The maximum is kept on the raw scores; the scale (times log2 e)
    // enters the exponent through one fused multiply-add: p = 2^(s*sc - m*sc).
    bool need_mask = (t * FA_BK + FA_BK - 1 > q_lo + qrow) || (p.window > 0 && t * FA_BK <= q_hi - p.window + 0);
    float mx[2] = {-INFINITY, -INFINITY};
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          int key = t * FA_BK + i * 8 + tig * 2 + (e & 1);
          int qp = (e >> 1) ? qpos_b : qpos_a;
          bool seen = key <= qp && (p.window == 0 || key > qp - p.window);
          if (!seen) s[i][e] = -INFINITY;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      mx[0] = fmaxf(mx[0], fmaxf(s[i][0], s[i][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[i][2], s[i][3]));
    }
    float corr[2], msc[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      float m_new = fmaxf(m[r], mx[r]);
      float m_fin = (m_new == -INFINITY) ? 0.f : m_new;        // nothing seen yet: every s is -inf, p = 0
      corr[r] = ex2_approx((m[r] - m_fin) * sc);               // m[r] = -inf gives 0
      msc[r] = m_fin * sc;
      m[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[4][4];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      float e0 = ex2_approx(fmaf(s[i][0], sc, -msc[0]));
      float e1 = ex2_approx(fmaf(s[i][1], sc, -msc[0]));
      float e2 = ex2_approx(fmaf(s[i][2], sc, -msc[1]));
      float e3 = ex2_approx(fmaf(s[i][3], sc, -msc[1]));
      rs[0] += e0 + e1;
      rs[1] += e2 + e3;
      pf[i >> 1][(i & 1) * 2] = pack_bf16(e0, e1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(e2, e3);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) l[r] = l[r] * corr[r] + rs[r];   // per-thread partial row sums; reduced at the end
#pragma unroll
    for (int i = 0; i < HD / 8; i++) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; dp++) {
        uint32_t b0, b1, b2, b3;
        int vrow = kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
        ldsm_x4_t(vbase + tile_off<HD>(vrow, dp * 2 + (lane >> 4)), b0, b1, b2, b3);
        mma16816(o[2 * dp], pf[kk], b0, b1);
        mma16816(o[2 * dp + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();       // everyone is done with `buf` before the next iteration's load overwrites it
  }
  cp_async_wait<0>();
  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; r++) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  float inv0 = l[0] > 0.f ? 1.f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.f / l[1] : 0.f;
  int ra = qrow + gid, rb = ra + 8;
  bf16* oa = p.out + (size_t)(row0 + r0 + ra) * ((size_t)p.H * HD) + (size_t)h * HD;
  bf16* ob = p.out + (size_t)(row0 + r0 + rb) * ((size_t)p.H * HD) + (size_t)h * HD;
#pragma unroll
  for (int i = 0; i < HD / 8; i++) {
    int col = i * 8 + tig * 2;
    if (ra < nq) *(uint32_t*)(oa + col) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    if (rb < nq) *(uint32_t*)(ob + col) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
}

template <int HD>
static int fa_launch(const FaArgs& a, int B, int max_new, cudaStream_t stream) {
  constexpr size_t smem = FA_BQ * HD * 2 + 4 * FA_BK * HD * 2;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid(a.H, (max_new + FA_BQ - 1) / FA_BQ, B);
  attn_prefill_kernel<HD><<<grid, FA_THREADS, smem, stream>>>(a);
  SLLM_RETURN_LAST();
}

SLLM_EXPORT int sllm_attn_prefill_bf16(const void* q, int q_ld, void* out, const int* seq_start, const int* seq_pos0,
                                       const int* block_table, int max_pages, const void* kpages, const void* vpages,
                                       int B, int max_new, int H, int G, int hd, int window, float scale,
                                       cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (G < 1 || H % G != 0 || (q_ld & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 3)) return SLLM_ERR_ARG;
  FaArgs a{(const bf16*)q, q_ld, (bf16*)out, seq_start, seq_pos0, block_table, max_pages, (const bf16*)kpages,
           (const bf16*)vpages, H, G, window, scale};
  if (hd == 64) return fa_launch<64>(a, B, max_new, stream);
  if (hd == 128) return fa_launch<128>(a, B, max_new, stream);
  return SLLM_ERR_ARG;
}

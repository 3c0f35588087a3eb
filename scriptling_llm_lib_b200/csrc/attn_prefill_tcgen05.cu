// Causal grouped-query attention of a prompt step over the paged cache on tcgen05 tensor cores
// (bfloat16, head width 64 or 128; a head of 128 is two 64-wide swizzled blocks side by side in
// shared memory for Q, K and V alike, and O takes 128 columns of tensor memory).
//
// Common to both head widths. A query tile is 128 consecutive queries of one sequence and one
// query head. Blocks stay and walk work items that are numbered longest first (heads fastest, then
// the sequences, query tiles from the last to the first) and dealt in rows that run forth and back
// (block k takes items k, 2G-1-k, 2G+k, ... of G blocks), so that a block's long items are paired
// with short ones and every block ends at about the same time; barriers, tensor memory and the
// key/value ring live across a block's items. One warp fetches the query tile and, page by page,
// the keys and values of the sequence with TMA (128-byte swizzle, no multicast) -- the pages are
// found through the block table, this step's own keys were written to the cache before. One thread
// issues the products: S = Q K^T (128 x 64, float, in tensor memory) and O += P V. Four softmax
// warps: thread = query row = tensor-memory lane, so a row's maximum and sum need no shuffles. They
// read a row of S, keep a reference maximum and the running sum (base 2, scale folded into one
// FFMA; the FFMAs and the sums two floats to an instruction) and write the probabilities as bfloat16 pairs back into tensor memory, from where P V takes
// them as its A operand: P never passes through shared memory, whose bandwidth (128 bytes a clock)
// the operand reads of these narrow products and the TMA writes already use to the full. O stays in
// tensor memory and is accumulated by the tensor core itself; the softmax threads rescale it (read,
// multiply, write back) only when a row's maximum has grown by more than 2^8 since its reference
// was set -- probabilities then stay below 2^8, and the final division by the row sum makes the
// result the same as with an exact running maximum (float32_ops.go:190-235; key j is seen by the
// query at position p when j <= p, and with a window only when j > p - window). The hand-over
// between the roles is by mbarriers; every wait is bounded (2 s), after which the kernel raises
// *err, drains its own TMA copies, frees its tensor memory and returns.
//
// Head width 64 (attn_prefill_tc_kernel): one query tile per work item, two blocks per SM, two S
// buffers and two P buffers beside O in the block's 256 columns.
//
// Head width 128 (attn_prefill_pair_kernel): a page of keys and values is 32 KB, and fetching it for
// every query tile by itself is what bounds the first form there (L2 to shared memory). So one block
// per SM works on a pair of query tiles that read the same keys and values -- two query heads of one
// key/value group on the same 128 queries where the group has an even number of heads, else two
// consecutive query tiles of one head -- and fetches each page once for both. Either tile of the
// pair has its own issuing thread, softmax warps, barriers and 256 columns (one S buffer, two P
// buffers, O); the two share the query/key/value fetches and the key/value ring, whose stage is
// free when both have used it.
#include "tcgen05.cuh"

#define FT_BQ 128
#define FT_BK 64           // = SLLM_PAGE
#define FT_THREADS 192       // warp 0: TMA, warp 1: MMA, warps 2-5: softmax (thread = query row)
#define FT_LOG2E 1.4426950408889634f

struct FtArgs {
  bf16* out;            // [T, H*64]
  const int* seq_start; // [B+1]
  const int* seq_pos0;  // [B]
  const int* block_table;
  int max_pages;
  int H, G, window;
  float scale;
  int* err;
  int n_qt, n_seqs, n_items;   // query tiles per sequence (of the longest), sequences, work items
  int pair_heads;              // pair kernel: 1: an item is heads 2i, 2i+1 on one query tile; 0: query tiles 2i, 2i+1 of one head
};

// What a block works on in its r-th round.
struct FtItem {
  int b, h, g, row0, r0, nq, pos0, t_lo, t_hi, n_tiles, q_hi;
  bool valid;           // false: past the end of a shorter sequence -- nothing to do
};
__device__ __forceinline__ bool ft_item(const FtArgs& p, int round, FtItem& it) {
  int G = gridDim.x;
  int idx = round * G + ((round & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
  if (idx >= p.n_items) return false;
  it.h = idx % p.H;
  int rest = idx / p.H;
  it.b = rest % p.n_seqs;
  int qt = p.n_qt - 1 - rest / p.n_seqs;
  it.row0 = p.seq_start[it.b];
  int S = p.seq_start[it.b + 1] - it.row0;
  it.r0 = qt * FT_BQ;
  it.valid = it.r0 < S;
  it.nq = min(FT_BQ, S - it.r0);
  it.pos0 = p.seq_pos0[it.b];
  it.g = it.h / (p.H / p.G);
  int q_lo = it.pos0 + it.r0;
  it.q_hi = it.pos0 + it.r0 + it.nq - 1;
  int k_first = p.window > 0 ? max(0, q_lo - p.window + 1) : 0;
  it.t_lo = k_first / FT_BK;
  it.t_hi = it.q_hi / FT_BK;
  it.n_tiles = it.t_hi - it.t_lo + 1;
  return true;
}

__device__ __forceinline__ float ft_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ft_max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
// two floats at once: d = a * b + c and d = a + b on pairs held in 64-bit registers
__device__ __forceinline__ uint64_t ft_pack2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void ft_unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ft_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t ft_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A's row m in lane m, two bfloat16 of K per 32-bit column
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

template <int FT_HD, int FT_STAGES>
__global__ void __launch_bounds__(FT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, FtArgs p, uint32_t smem_bytes) {
  constexpr uint32_t Q_BYTES = FT_BQ * FT_HD * 2, KV_BYTES = FT_BK * FT_HD * 2;
  static_assert(FT_HD == 64, "S0, S1, O and two P buffers fill the 256 columns of a block at head width 64");
  constexpr uint32_t P_COL0 = 192, P_STEP = 32;
  constexpr uint32_t QA = FT_BQ * 128, KA = FT_BK * 128;       // bytes of one 64-wide block of Q and of a K or V page
  constexpr int NA = FT_HD / 64;                               // such blocks per head
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // [Q][K stages][V stages][barriers]
  const uint32_t sQ = smem_u32(smem), sK = sQ + Q_BYTES, sV = sK + FT_STAGES * KV_BYTES;
  uint64_t* bars = (uint64_t*)(smem + Q_BYTES + 2 * FT_STAGES * KV_BYTES);
  // q_full, kv_full[ST], kv_empty[ST], s_full[2], p_full[2], o_full[2], q_empty. The barriers of S, P and O
  // come in pairs, one for the tiles of each parity: a waiter is then never more than one phase behind.
  const uint32_t b_qfull = smem_u32(bars), b_kvfull = b_qfull + 8, b_kvempty = b_kvfull + 8 * FT_STAGES,
                 b_sfull = b_kvempty + 8 * FT_STAGES, b_pfull = b_sfull + 16, b_ofull = b_pfull + 16, b_qempty = b_ofull + 16;
  uint32_t* tmem_slot = (uint32_t*)(bars + 1 + 2 * FT_STAGES + 2 + 2 + 2 + 1);
  volatile int* abort = (volatile int*)(tmem_slot + 1);
  if ((uint8_t*)(abort + 1) > smem_raw + smem_bytes) {      // the 1 KB alignment took more than the launch left room for
    if (threadIdx.x == 0) atomicExch(p.err, 3);
    return;
  }

  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int s = 0; s < FT_STAGES; s++) { mbar_init(b_kvfull + 8 * s, 1); mbar_init(b_kvempty + 8 * s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(b_sfull + 8 * a, 1); mbar_init(b_pfull + 8 * a, 4); mbar_init(b_ofull + 8 * a, 1); }
    mbar_init(b_qempty, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;          // columns: S0 0-63, S1 64-127, O 128-191 (one column per dim), P0 192-223, P1 224-255

  // Every role walks the same items in the same order and counts tiles (J) and items (I) by itself; a
  // barrier's phase follows from those counts, so nothing is set up again between items.
  if (warp == 0) {
    if (lane == 0) {
      int J = 0, I = 0;
      FtItem it;
      bool ok = true;
      for (int round = 0; ok && ft_item(p, round, it); round++) {
        if (!it.valid) continue;
        const int* bt = p.block_table + (size_t)it.b * p.max_pages;
        // the products of the last item that read Q are done
        if (!mbar_wait(b_qempty, (I & 1) ^ 1, abort)) break;
        mbar_expect_tx(b_qfull, Q_BYTES);
#pragma unroll
        for (int a = 0; a < NA; a++) tma_load_2d(sQ + a * QA, &map_q, it.h * FT_HD + 64 * a, it.row0 + it.r0, b_qfull);
        I++;
        for (int j = 0; j < it.n_tiles; j++) {
          int s = J % FT_STAGES;
          if (!mbar_wait(b_kvempty + 8 * s, ((J / FT_STAGES) & 1) ^ 1, abort)) { ok = false; break; }
          int page = bt[it.t_lo + j];
          int krow = (page * p.G + it.g) * FT_BK;
          mbar_expect_tx(b_kvfull + 8 * s, 2 * KV_BYTES);
#pragma unroll
          for (int a = 0; a < NA; a++) {
            tma_load_2d(sK + s * KV_BYTES + a * KA, &map_k, 64 * a, krow, b_kvfull + 8 * s);
            tma_load_2d(sV + s * KV_BYTES + a * KA, &map_v, 64 * a, krow, b_kvfull + 8 * s);
          }
          J++;
        }
      }
      if (*abort) {            // let the copies that are under way land before the block leaves
        volatile int never = 0;
        if (I > 0) mbar_wait(b_qfull, (I - 1) & 1, &never);
        for (int j = max(0, J - FT_STAGES); j < J; j++) mbar_wait(b_kvfull + 8 * (j % FT_STAGES), (j / FT_STAGES) & 1, &never);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FT_BQ, FT_BK);          // S = Q K^T: both K-major
      constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(FT_BQ, FT_HD);      // O = P V: V is MN-major (dims contiguous)
      int J0 = 0, I = 0;
      FtItem it;
      bool ok = true;
      for (int round = 0; ok && ft_item(p, round, it); round++) {
        if (!it.valid) continue;
        const int n_tiles = it.n_tiles;
        ok = mbar_wait(b_qfull, I & 1, abort);
        I++;
        auto issue_s = [&](int j) -> bool {
          int Jg = J0 + j, s = Jg % FT_STAGES, a = Jg & 1;
          if (!mbar_wait(b_kvfull + 8 * s, (Jg / FT_STAGES) & 1, abort)) return false;
          // S(Jg) takes the place of S(Jg-2), which the softmax threads have read (their P(Jg-2) was waited for)
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int k = 0; k < FT_HD / 16; k++)      // 16 dims a step: four steps in each 64-wide block
            umma_bf16(tmem_base + a * 64, umma_desc_sw128(sQ + (k >> 2) * QA + (k & 3) * 32),
                      umma_desc_sw128(sK + s * KV_BYTES + (k >> 2) * KA + (k & 3) * 32), idesc_s, k ? 1u : 0u);
          umma_commit(b_sfull + 8 * a);
          if (j == n_tiles - 1) umma_commit(b_qempty);     // the item's last product that reads Q
          return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < n_tiles && ok; j++) {
          if (j + 1 < n_tiles) { ok = issue_s(j + 1); if (!ok) break; }
          int Jg = J0 + j, s = Jg % FT_STAGES, a = Jg & 1;
          ok = mbar_wait(b_pfull + 8 * a, (Jg >> 1) & 1, abort);   // P of tile j is written, and O has been rescaled if it had to be
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int k = 0; k < FT_BK / 16; k++)
            umma_bf16_ta(tmem_base + 128, tmem_base + P_COL0 + a * P_STEP + k * 8, umma_desc_sw128_mn(sV + s * KV_BYTES + k * 2048, NA > 1 ? KA : 0),
                         idesc_o, (j | k) ? 1u : 0u);
          umma_commit(b_ofull + 8 * a);
          umma_commit(b_kvempty + 8 * s);
        }
        J0 += n_tiles;
      }
    }
  } else {
    const int q = warp & 3;                        // tensor-memory quarter of this warp
    const int r = q * 32 + lane;                   // query row of this thread in the tile
    const float sc = p.scale * FT_LOG2E;
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
    int J0 = 0;
    FtItem it;
    bool ok = true;
    for (int round = 0; ok && ft_item(p, round, it); round++) {
    if (!it.valid) continue;
    const int n_tiles = it.n_tiles, t_lo = it.t_lo, t_hi = it.t_hi, q_hi = it.q_hi, nq = it.nq, row0 = it.row0, r0 = it.r0, h = it.h;
    const int qpos = it.pos0 + r0 + r;
    float m_ref = -INFINITY, l = 0.f;              // reference maximum (raw score units) and sum relative to it
    for (int j = 0; j < n_tiles && ok; j++) {
      const int Jg = J0 + j;
      int a = Jg & 1, t = t_lo + j;
      ok = mbar_wait(b_sfull + 8 * a, (Jg >> 1) & 1, abort);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t s0[32], s1[32];
      tmem_ld32(t_lane + a * 64, s0);
      tmem_ld32(t_lane + a * 64 + 32, s1);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      // ---- mask, row maximum (raw scores; four independent chains)
      bool need_mask = (t * FT_BK + FT_BK - 1 > qpos) || (p.window > 0 && t * FT_BK <= qpos - p.window);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; i++) {
          int k0 = t * FT_BK + i, k1 = k0 + 32;
          if (!(k0 <= qpos && (p.window == 0 || k0 > qpos - p.window))) s0[i] = 0xff800000u;   // -inf
          if (!(k1 <= qpos && (p.window == 0 || k1 > qpos - p.window))) s1[i] = 0xff800000u;
        }
      }
      float mxa = ft_max3(__uint_as_float(s0[0]), __uint_as_float(s0[1]), __uint_as_float(s0[2]));
      float mxb = ft_max3(__uint_as_float(s0[3]), __uint_as_float(s0[4]), __uint_as_float(s0[5]));
      float mxc = ft_max3(__uint_as_float(s1[0]), __uint_as_float(s1[1]), __uint_as_float(s1[2]));
      float mxd = ft_max3(__uint_as_float(s1[3]), __uint_as_float(s1[4]), __uint_as_float(s1[5]));
#pragma unroll
      for (int i = 6; i < 32; i += 4) {      // 6..29, then 30, 31
        if (i + 3 < 32) {
          mxa = ft_max3(mxa, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
          mxb = ft_max3(mxb, __uint_as_float(s0[i + 2]), __uint_as_float(s0[i + 3]));
          mxc = ft_max3(mxc, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
          mxd = ft_max3(mxd, __uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3]));
        } else {
          mxa = ft_max3(mxa, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
          mxc = ft_max3(mxc, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
        }
      }
      float mx = fmaxf(ft_max3(mxa, mxb, mxc), mxd);
      // ---- move the reference maximum only when the row's maximum has outgrown it by 2^8
      bool grow = mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * sc > 8.0f);
      if (__any_sync(0xffffffffu, grow)) {
        float factor = grow ? ((m_ref == -INFINITY) ? 0.f : ft_ex2((m_ref - mx) * sc)) : 1.f;
        if (j >= 1) {
          // O holds the products of tiles 0..j-1: they must be complete before it is rewritten
          ok = mbar_wait(b_ofull + 8 * (a ^ 1), ((Jg - 1) >> 1) & 1, abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint32_t v[32];
#pragma unroll 1
          for (int c0 = 0; c0 < FT_HD; c0 += 32) {
            tmem_ld32(t_lane + 128 + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
            tmem_st32(t_lane + 128 + c0, v);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        l *= factor;
        if (grow) m_ref = mx;
      }
      float msc = (m_ref == -INFINITY) ? 0.f : m_ref * sc;
      uint64_t rs2 = 0ull;                          // two partial sums side by side
      const uint64_t sc2 = ft_pack2(sc, sc), nm2 = ft_pack2(-msc, -msc);
      uint32_t pk[32];                              // 64 probabilities as bfloat16 pairs: keys 2i, 2i+1
#pragma unroll
      for (int i = 0; i < 16; i++) {
        float x0, x1, x2, x3;
        ft_unpack2(ft_fma2(ft_pack2(__uint_as_float(s0[2 * i]), __uint_as_float(s0[2 * i + 1])), sc2, nm2), x0, x1);
        ft_unpack2(ft_fma2(ft_pack2(__uint_as_float(s1[2 * i]), __uint_as_float(s1[2 * i + 1])), sc2, nm2), x2, x3);
        float e0 = ft_ex2(x0), e1 = ft_ex2(x1), e2 = ft_ex2(x2), e3 = ft_ex2(x3);
        rs2 = ft_add2(rs2, ft_add2(ft_pack2(e0, e1), ft_pack2(e2, e3)));
        __nv_bfloat162 lo = __floats2bfloat162_rn(e0, e1), hi = __floats2bfloat162_rn(e2, e3);
        pk[i] = *(uint32_t*)&lo;
        pk[16 + i] = *(uint32_t*)&hi;
      }
      {
        float ra, rb;
        ft_unpack2(rs2, ra, rb);
        l += ra + rb;
      }
      // ---- P into tensor memory. The product that read this buffer's last P, two tiles ago, is complete:
      // it was issued before S(Jg), and the commit that announced S(Jg) covers every product issued before it.
      if (t == t_hi) {
        // keys of the last page beyond the last query's position hold whatever the page held before:
        // their probabilities are zero, but 0 * NaN is NaN, so their value rows are cleared
        int s = Jg % FT_STAGES, n_valid = q_hi + 1 - t * FT_BK;
        ok = mbar_wait(b_kvfull + 8 * s, (Jg / FT_STAGES) & 1, abort);
        if (!ok) break;
        for (int e = (warp - 2) * 32 + lane; e < (FT_BK - n_valid) * 8 * NA; e += 128) {
          int blk = e / ((FT_BK - n_valid) * 8), e1 = e % ((FT_BK - n_valid) * 8);
          int row = n_valid + e1 / 8, c = e1 % 8;
          *(uint4*)(smem + Q_BYTES + FT_STAGES * KV_BYTES + s * KV_BYTES + blk * KA + row * 128 + ((c ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      tmem_st32(t_lane + P_COL0 + a * P_STEP, pk);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(b_pfull + 8 * a);
    }
    if (ok) ok = mbar_wait(b_ofull + 8 * ((J0 + n_tiles - 1) & 1), ((J0 + n_tiles - 1) >> 1) & 1, abort);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (size_t)(row0 + r0 + r) * ((size_t)p.H * FT_HD) + (size_t)h * FT_HD;
#pragma unroll 1
      for (int c0 = 0; c0 < FT_HD; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(t_lane + 128 + c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (r < nq) {
#pragma unroll
          for (int c = 0; c < 4; c++) {
            uint4 w;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(v[8 * c]) * inv, __uint_as_float(v[8 * c + 1]) * inv);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2]) * inv, __uint_as_float(v[8 * c + 3]) * inv);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 4]) * inv, __uint_as_float(v[8 * c + 5]) * inv);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 6]) * inv, __uint_as_float(v[8 * c + 7]) * inv);
            w.x = *(uint32_t*)&p0; w.y = *(uint32_t*)&p1; w.z = *(uint32_t*)&p2; w.w = *(uint32_t*)&p3;
            *(uint4*)(dst + c0 + 8 * c) = w;
          }
        }
      }
    }
    // the rows of O are read (the loads above were waited for) before this thread signals the next item's first P
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    J0 += n_tiles;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
  if (threadIdx.x == 0 && *abort) atomicExch(p.err, 2);
}

// ------------------------------------------------------------------ pairs of query tiles (head width 128)
#define FP_THREADS 384       // warp 0: TMA, warps 1-2: the issuing thread of either tile, warp 3: nothing; warps 4-7 and 8-11: softmax of either tile

// One query tile of a pair.
struct FpTile {
  int h, r0, nq, q_hi, t_lo, t_hi, n_tiles;
  bool valid;           // false: past the end of the sequence -- nothing to do
};
// What a block works on in its r-th round.
struct FpItem {
  int b, g, row0, pos0, seq_end, T_lo, n_union;
  FpTile sub[2];
  bool valid;
};
__device__ __forceinline__ void fp_tile(const FtArgs& p, FpTile& s, int h, int qt, int S, int pos0) {
  s.h = h;
  s.r0 = qt * FT_BQ;
  s.valid = s.r0 < S;
  s.nq = min(FT_BQ, S - s.r0);
  int q_lo = pos0 + s.r0;
  s.q_hi = pos0 + s.r0 + s.nq - 1;
  int k_first = p.window > 0 ? max(0, q_lo - p.window + 1) : 0;
  s.t_lo = k_first / FT_BK;
  s.t_hi = s.q_hi / FT_BK;
  s.n_tiles = s.t_hi - s.t_lo + 1;
}
__device__ __forceinline__ bool fp_item(const FtArgs& p, int round, FpItem& it) {
  int G = gridDim.x;
  int idx = round * G + ((round & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
  if (idx >= p.n_items) return false;
  int h0, h1, qt0, qt1, rest;
  if (p.pair_heads) {
    int H2 = p.H >> 1;
    h0 = 2 * (idx % H2);
    h1 = h0 + 1;
    rest = idx / H2;
    qt0 = qt1 = p.n_qt - 1 - rest / p.n_seqs;
  } else {
    h0 = h1 = idx % p.H;
    rest = idx / p.H;
    int n_qp = (p.n_qt + 1) >> 1;
    qt0 = 2 * (n_qp - 1 - rest / p.n_seqs);
    qt1 = qt0 + 1;
  }
  it.b = rest % p.n_seqs;
  it.row0 = p.seq_start[it.b];
  int S = p.seq_start[it.b + 1] - it.row0;
  it.pos0 = p.seq_pos0[it.b];
  it.seq_end = it.pos0 + S - 1;
  it.g = h0 / (p.H / p.G);
  fp_tile(p, it.sub[0], h0, qt0, S, it.pos0);
  fp_tile(p, it.sub[1], h1, qt1, S, it.pos0);
  it.valid = it.sub[0].valid;                      // the second tile of a pair is never valid without the first
  int lo = it.sub[0].t_lo, hi = it.sub[0].t_hi;
  if (it.sub[1].valid) { lo = min(lo, it.sub[1].t_lo); hi = max(hi, it.sub[1].t_hi); }
  it.T_lo = lo;
  it.n_union = hi - lo + 1;                        // key tiles T_lo ... T_lo + n_union - 1; every one is in either tile's range
  return true;
}
__device__ __forceinline__ bool fp_active(const FpTile& s, int t) { return s.valid && t >= s.t_lo && t <= s.t_hi; }

// maximum of a row's 64 scores, four chains of three-input maxima
__device__ __forceinline__ float ft_rowmax(const uint32_t (&s)[64]) {
  float m[4];
#pragma unroll
  for (int c = 0; c < 4; c++) m[c] = ft_max3(__uint_as_float(s[16 * c]), __uint_as_float(s[16 * c + 1]), __uint_as_float(s[16 * c + 2]));
#pragma unroll
  for (int i = 3; i < 15; i += 2)
#pragma unroll
    for (int c = 0; c < 4; c++) m[c] = ft_max3(m[c], __uint_as_float(s[16 * c + i]), __uint_as_float(s[16 * c + i + 1]));
#pragma unroll
  for (int c = 0; c < 4; c++) m[c] = fmaxf(m[c], __uint_as_float(s[16 * c + 15]));
  return fmaxf(ft_max3(m[0], m[1], m[2]), m[3]);
}
// scores of keys the query at qpos does not see become -inf (tile t holds keys 64 t ... 64 t + 63)
__device__ __forceinline__ void ft_mask(uint32_t (&s)[64], int t, int qpos, int window) {
  bool need = (t * FT_BK + FT_BK - 1 > qpos) || (window > 0 && t * FT_BK <= qpos - window);
  if (need) {
#pragma unroll
    for (int i = 0; i < 64; i++) {
      int k = t * FT_BK + i;
      if (!(k <= qpos && (window == 0 || k > qpos - window))) s[i] = 0xff800000u;   // -inf
    }
  }
}
__device__ __forceinline__ void ft_ld64(uint32_t taddr, uint32_t (&s)[64]) {
  tmem_ld32(taddr, *(uint32_t(*)[32])&s[0]);
  tmem_ld32(taddr + 32, *(uint32_t(*)[32])&s[32]);
}

template <int FT_HD, int FT_STAGES>
__global__ void __launch_bounds__(FP_THREADS, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, FtArgs p, uint32_t smem_bytes) {
  constexpr uint32_t Q_BYTES = FT_BQ * FT_HD * 2, KV_BYTES = FT_BK * FT_HD * 2;
  constexpr uint32_t QA = FT_BQ * 128, KA = FT_BK * 128;       // bytes of one 64-wide block of Q and of a K or V page
  constexpr int NA = FT_HD / 64;                               // such blocks per head
  // tensor-memory columns of one tile of the pair (256): a head of 64 has S0 0-63, S1 64-127, O 128-191, P0 192-223,
  // P1 224-255; a head of 128, whose O takes 128-255, has one S buffer 0-63 and P0 64-95, P1 96-127
  constexpr int NBUF = FT_HD > 64 ? 1 : 2;       // S buffers; the next tile's S is issued while a tile's softmax runs
  constexpr uint32_t P_COL0 = FT_HD > 64 ? 64 : 192, P_STEP = 32, SUB_COLS = 256;
  static_assert(FT_STAGES >= 3, "the key/value ring must hold the tile whose S is issued ahead");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // [Q of either tile][K stages][V stages][barriers]
  const uint32_t sQ = smem_u32(smem), sK = sQ + 2 * Q_BYTES, sV = sK + FT_STAGES * KV_BYTES;
  uint64_t* bars = (uint64_t*)(smem + 2 * Q_BYTES + 2 * FT_STAGES * KV_BYTES);
  // q_full, q_empty, kv_full[ST], kv_empty[ST], then for either tile of the pair s_full[2], s_empty[2], p_full[2],
  // o_full[2]. The barriers of P and O come in pairs, one for the tiles of each parity, those of S one per
  // buffer: a waiter is then never more than one phase behind.
  const uint32_t b_qfull = smem_u32(bars), b_qempty = b_qfull + 8, b_kvfull = b_qempty + 8, b_kvempty = b_kvfull + 8 * FT_STAGES,
                 b_sub = b_kvempty + 8 * FT_STAGES;      // + x * 64: s_full[2], s_empty[2], p_full[2], o_full[2]
  constexpr uint32_t SUB_BARS = 64, B_SEMPTY = 16, B_PFULL = 32, B_OFULL = 48;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 + 2 * FT_STAGES + 16);
  volatile int* abort = (volatile int*)(tmem_slot + 1);
  if ((uint8_t*)(abort + 1) > smem_raw + smem_bytes) {      // the 1 KB alignment took more than the launch left room for
    if (threadIdx.x == 0) atomicExch(p.err, 3);
    return;
  }

  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    mbar_init(b_qempty, 2);                        // either issuing thread arrives
    for (int s = 0; s < FT_STAGES; s++) { mbar_init(b_kvfull + 8 * s, 1); mbar_init(b_kvempty + 8 * s, 2); }
    for (int x = 0; x < 2; x++)
      for (int a = 0; a < 2; a++) {
        mbar_init(b_sub + SUB_BARS * x + 8 * a, 1);
        mbar_init(b_sub + SUB_BARS * x + B_SEMPTY + 8 * a, 4);
        mbar_init(b_sub + SUB_BARS * x + B_PFULL + 8 * a, 4);
        mbar_init(b_sub + SUB_BARS * x + B_OFULL + 8 * a, 1);
      }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // Every role walks the same items in the same order and counts by itself the key tiles fetched (JU),
  // the tiles its query tile of the pair has taken (J) and the items (I); a barrier's phase follows from
  // those counts, so nothing is set up again between items.
  if (warp < 4) {
    if (warp == 0) {
      if (lane == 0) {
        int JU = 0, I = 0;
        FpItem it;
        bool ok = true;
        for (int round = 0; ok && fp_item(p, round, it); round++) {
          if (!it.valid) continue;
          const int* bt = p.block_table + (size_t)it.b * p.max_pages;
          // the products of the last item that read Q are done
          if (!mbar_wait(b_qempty, (I & 1) ^ 1, abort)) break;
          mbar_expect_tx(b_qfull, it.sub[1].valid ? 2 * Q_BYTES : Q_BYTES);
#pragma unroll
          for (int x = 0; x < 2; x++)
            if (it.sub[x].valid) {
#pragma unroll
              for (int a = 0; a < NA; a++)
                tma_load_2d(sQ + x * Q_BYTES + a * QA, &map_q, it.sub[x].h * FT_HD + 64 * a, it.row0 + it.sub[x].r0, b_qfull);
            }
          I++;
          for (int u = 0; u < it.n_union; u++) {
            int s = JU % FT_STAGES;
            if (!mbar_wait(b_kvempty + 8 * s, ((JU / FT_STAGES) & 1) ^ 1, abort)) { ok = false; break; }
            int page = bt[it.T_lo + u];
            int krow = (page * p.G + it.g) * FT_BK;
            mbar_expect_tx(b_kvfull + 8 * s, 2 * KV_BYTES);
#pragma unroll
            for (int a = 0; a < NA; a++) {
              tma_load_2d(sK + s * KV_BYTES + a * KA, &map_k, 64 * a, krow, b_kvfull + 8 * s);
              tma_load_2d(sV + s * KV_BYTES + a * KA, &map_v, 64 * a, krow, b_kvfull + 8 * s);
            }
            JU++;
          }
        }
        if (*abort) {            // let the copies that are under way land before the block leaves
          volatile int never = 0;
          if (I > 0) mbar_wait(b_qfull, (I - 1) & 1, &never);
          for (int j = max(0, JU - FT_STAGES); j < JU; j++) mbar_wait(b_kvfull + 8 * (j % FT_STAGES), (j / FT_STAGES) & 1, &never);
        }
      }
    } else if (warp <= 2) {
      if (lane == 0) {
        const int x = warp - 1;                    // this thread issues the products of one tile of the pair
        constexpr uint32_t idesc_s = umma_idesc_bf16(FT_BQ, FT_BK);          // S = Q K^T: both K-major
        constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(FT_BQ, FT_HD);      // O = P V: V is MN-major (dims contiguous)
        int JU0 = 0, I = 0, J0 = 0;
        FpItem it;
        bool ok = true;
        for (int round = 0; ok && fp_item(p, round, it); round++) {
          if (!it.valid) continue;
          const int n_union = it.n_union;
          const FpTile sub = it.sub[x];
          ok = mbar_wait(b_qfull, I & 1, abort);
          I++;
          auto issue_s = [&](int u) -> bool {
            const int JUg = JU0 + u, s = JUg % FT_STAGES, t = it.T_lo + u;
            if (!mbar_wait(b_kvfull + 8 * s, (JUg / FT_STAGES) & 1, abort)) return false;
            if (fp_active(sub, t)) {
              const int Jg = J0 + t - sub.t_lo, sb = Jg % NBUF;
              // S(Jg) takes the place of S(Jg - NBUF), which the softmax threads have taken into their registers: with
              // two buffers their P(Jg - 2) was waited for; the single buffer has a barrier for it
              if (NBUF == 1 && !mbar_wait(b_sub + SUB_BARS * x + B_SEMPTY + 8 * sb, ((Jg / NBUF) & 1) ^ 1, abort)) return false;
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
              for (int k = 0; k < FT_HD / 16; k++)      // 16 dims a step: four steps in each 64-wide block
                umma_bf16(tmem_base + x * SUB_COLS + sb * 64, umma_desc_sw128(sQ + x * Q_BYTES + (k >> 2) * QA + (k & 3) * 32),
                          umma_desc_sw128(sK + s * KV_BYTES + (k >> 2) * KA + (k & 3) * 32), idesc_s, k ? 1u : 0u);
              umma_commit(b_sub + SUB_BARS * x + 8 * sb);
            }
            if (u == n_union - 1) umma_commit(b_qempty);     // the item's last products that read Q
            return true;
          };
          if (ok) ok = issue_s(0);
          for (int u = 0; u < n_union && ok; u++) {
            if (u + 1 < n_union) { ok = issue_s(u + 1); if (!ok) break; }
            const int JUg = JU0 + u, s = JUg % FT_STAGES, t = it.T_lo + u;
            if (fp_active(sub, t)) {
              const int j = t - sub.t_lo, Jg = J0 + j, a = Jg & 1;
              ok = mbar_wait(b_sub + SUB_BARS * x + B_PFULL + 8 * a, (Jg >> 1) & 1, abort);   // P of this tile is written, and O has been rescaled if it had to be
              if (!ok) break;
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
              for (int k = 0; k < FT_BK / 16; k++)
                umma_bf16_ta(tmem_base + x * SUB_COLS + 128, tmem_base + x * SUB_COLS + P_COL0 + a * P_STEP + k * 8,
                             umma_desc_sw128_mn(sV + s * KV_BYTES + k * 2048, NA > 1 ? KA : 0), idesc_o, (j | k) ? 1u : 0u);
              umma_commit(b_sub + SUB_BARS * x + B_OFULL + 8 * a);
            }
            if (!ok) break;
            umma_commit(b_kvempty + 8 * s);
          }
          JU0 += n_union;
          if (sub.valid) J0 += sub.n_tiles;
        }
      }
    }
  } else {
    const int x = (warp >> 2) - 1;                 // which tile of the pair
    const int q = warp & 3;                        // tensor-memory quarter of this warp
    const int r = q * 32 + lane;                   // query row of this thread in the tile
    const float sc = p.scale * FT_LOG2E;
    const uint32_t t_lane = tmem_base + x * SUB_COLS + ((uint32_t)(q * 32) << 16);
    const uint32_t b_sfull = b_sub + SUB_BARS * x, b_sempty = b_sfull + B_SEMPTY, b_pfull = b_sfull + B_PFULL, b_ofull = b_sfull + B_OFULL;
    int J0 = 0, JU0 = 0;
    FpItem it;
    bool ok = true;
    for (int round = 0; ok && fp_item(p, round, it); round++) {
    if (!it.valid) continue;
    const FpTile sb = it.sub[x];
    const int n_union = it.n_union, T_lo = it.T_lo;
    if (sb.valid) {
    const int n_tiles = sb.n_tiles, t_lo = sb.t_lo, seq_end = it.seq_end;
    const int qpos = it.pos0 + sb.r0 + r;
    float m_ref = -INFINITY, l = 0.f;              // reference maximum (raw score units) and sum relative to it
    uint32_t s[64];
    float mx;
#pragma unroll 1
    for (int j = 0; j < n_tiles && ok; j++) {
      const int Jg = J0 + j;
      const int a = Jg & 1, t = t_lo + j, bf = Jg % NBUF;
      ok = mbar_wait(b_sfull + 8 * bf, (Jg / NBUF) & 1, abort);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      ft_ld64(t_lane + bf * 64, s);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (NBUF == 1) {                             // the one S buffer may take the next tile's scores
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(b_sempty + 8 * bf);
      }
      ft_mask(s, t, qpos, p.window);
      mx = ft_rowmax(s);
      // ---- move the reference maximum only when the row's maximum has outgrown it by 2^8
      bool grow = mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * sc > 8.0f);
      if (__any_sync(0xffffffffu, grow)) {
        float factor = grow ? ((m_ref == -INFINITY) ? 0.f : ft_ex2((m_ref - mx) * sc)) : 1.f;
        if (j >= 1) {
          // O holds the products of tiles 0..j-1: they must be complete before it is rewritten
          ok = mbar_wait(b_ofull + 8 * (a ^ 1), ((Jg - 1) >> 1) & 1, abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint32_t v[32];
#pragma unroll 1
          for (int c0 = 0; c0 < FT_HD; c0 += 32) {
            tmem_ld32(t_lane + 128 + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
            tmem_st32(t_lane + 128 + c0, v);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        l *= factor;
        if (grow) m_ref = mx;
      }
      const float msc = (m_ref == -INFINITY) ? 0.f : m_ref * sc;
      uint64_t rs2 = 0ull;                          // two partial sums side by side
      const uint64_t sc2 = ft_pack2(sc, sc), nm2 = ft_pack2(-msc, -msc);
      uint32_t pk[32];                              // 64 probabilities as bfloat16 pairs: keys 2i, 2i+1
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float x0, x1, x2, x3;
        ft_unpack2(ft_fma2(ft_pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), sc2, nm2), x0, x1);
        ft_unpack2(ft_fma2(ft_pack2(__uint_as_float(s[2 * i + 2]), __uint_as_float(s[2 * i + 3])), sc2, nm2), x2, x3);
        float e0 = ft_ex2(x0), e1 = ft_ex2(x1), e2 = ft_ex2(x2), e3 = ft_ex2(x3);
        rs2 = ft_add2(rs2, ft_add2(ft_pack2(e0, e1), ft_pack2(e2, e3)));
        __nv_bfloat162 lo = __floats2bfloat162_rn(e0, e1), hi = __floats2bfloat162_rn(e2, e3);
        pk[i] = *(uint32_t*)&lo;
        pk[i + 1] = *(uint32_t*)&hi;
      }
      {
        float ra, rb;
        ft_unpack2(rs2, ra, rb);
        l += ra + rb;
      }
      if (t * FT_BK + FT_BK - 1 > seq_end) {
        // keys of the sequence's last page beyond its last position hold whatever the page held before:
        // their probabilities are zero, but 0 * NaN is NaN, so their value rows are cleared -- by either
        // tile of the pair that takes this page, each before its own P V product (zeros over zeros harm nothing)
        const int JUg = JU0 + t - T_lo, st = JUg % FT_STAGES, n_valid = max(0, seq_end + 1 - t * FT_BK);
        ok = mbar_wait(b_kvfull + 8 * st, (JUg / FT_STAGES) & 1, abort);
        if (!ok) break;
        for (int e = q * 32 + lane; e < (FT_BK - n_valid) * 8 * NA; e += 128) {
          int blk = e / ((FT_BK - n_valid) * 8), e1 = e % ((FT_BK - n_valid) * 8);
          int row = n_valid + e1 / 8, c = e1 % 8;
          *(uint4*)(smem + 2 * Q_BYTES + FT_STAGES * KV_BYTES + st * KV_BYTES + blk * KA + row * 128 + ((c ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      // ---- P into tensor memory. The product that read this buffer's last P, two tiles ago, is complete:
      // it was issued before S(Jg), and the commit that announced S(Jg) covers every product issued before it.
      tmem_st32(t_lane + P_COL0 + a * P_STEP, pk);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(b_pfull + 8 * a);
    }
    if (ok) ok = mbar_wait(b_ofull + 8 * ((J0 + n_tiles - 1) & 1), ((J0 + n_tiles - 1) >> 1) & 1, abort);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (size_t)(it.row0 + sb.r0 + r) * ((size_t)p.H * FT_HD) + (size_t)sb.h * FT_HD;
#pragma unroll 1
      for (int c0 = 0; c0 < FT_HD; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(t_lane + 128 + c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (r < sb.nq) {
#pragma unroll
          for (int c = 0; c < 4; c++) {
            uint4 w;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(v[8 * c]) * inv, __uint_as_float(v[8 * c + 1]) * inv);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2]) * inv, __uint_as_float(v[8 * c + 3]) * inv);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 4]) * inv, __uint_as_float(v[8 * c + 5]) * inv);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 6]) * inv, __uint_as_float(v[8 * c + 7]) * inv);
            w.x = *(uint32_t*)&p0; w.y = *(uint32_t*)&p1; w.z = *(uint32_t*)&p2; w.w = *(uint32_t*)&p3;
            *(uint4*)(dst + c0 + 8 * c) = w;
          }
        }
      }
    }
    // the rows of O are read (the loads above were waited for) before this thread signals the next item's first P
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    J0 += n_tiles;
    }
    JU0 += n_union;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  if (threadIdx.x == 0 && *abort) atomicExch(p.err, 1000 * (int)blockIdx.x + *abort);
}

template <int HD, int STAGES>
static int ft_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FtArgs& a, dim3 grid,
                     cudaStream_t stream) {
  // what the kernel lays out after aligning to 1 KB, and the most two blocks can have on an SM
  constexpr size_t need = FT_BQ * HD * 2 + 2 * STAGES * FT_BK * HD * 2 + 256;
  constexpr size_t room = (233472 / 2 - 1024);
  constexpr size_t smem = need + 1024 <= room ? need + 1024 : room;     // the slack for the alignment, as far as it fits
  static_assert(need <= smem, "two blocks of this head width do not fit an SM");
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  attn_prefill_tc_kernel<HD, STAGES><<<grid, FT_THREADS, smem, stream>>>(mq, mk, mv, a, (uint32_t)smem);
  SLLM_RETURN_LAST();
}

template <int HD, int STAGES>
static int fp_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FtArgs& a, dim3 grid,
                     cudaStream_t stream) {
  // what the kernel lays out after aligning to 1 KB; one block on an SM
  constexpr size_t need = 2 * FT_BQ * HD * 2 + 2 * STAGES * FT_BK * HD * 2 + 256;
  constexpr size_t room = 232448;
  constexpr size_t smem = need + 1024 <= room ? need + 1024 : room;     // the slack for the alignment, as far as it fits
  static_assert(need <= smem, "the block of this head width does not fit an SM");
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_pair_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  attn_prefill_pair_kernel<HD, STAGES><<<grid, FP_THREADS, smem, stream>>>(mq, mk, mv, a, (uint32_t)smem);
  SLLM_RETURN_LAST();
}

// q: [T, q_ld] rotated queries (head h at columns h*hd); out: [T, H*hd]; kpages/vpages:
// [n_pages][G][64][hd] with n_pages the number of pages the storage holds; hd 64 or 128.
SLLM_EXPORT int sllm_attn_prefill_tc_bf16(const void* q, int q_ld, int T, void* out, const int* seq_start, const int* seq_pos0,
                                          const int* block_table, int max_pages, const void* kpages, const void* vpages,
                                          long long n_pages, int B, int max_new, int H, int G, int hd, int window, float scale,
                                          int* err, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if ((hd != 64 && hd != 128) || G < 1 || H % G != 0 || (q_ld & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)kpages & 15) || ((uintptr_t)vpages & 15))
    return SLLM_ERR_ARG;
  long long kv_rows = n_pages * G * FT_BK;
  if (kv_rows <= 0 || kv_rows > 0x7fffffffLL) return SLLM_ERR_ARG;
  CUtensorMap mq, mk, mv;
  int rc = tc_make_map(&mq, q, T, q_ld, q_ld, FT_BQ);
  if (rc) return rc;
  rc = tc_make_map(&mk, kpages, (int)kv_rows, hd, hd, FT_BK);
  if (rc) return rc;
  rc = tc_make_map(&mv, vpages, (int)kv_rows, hd, hd, FT_BK);
  if (rc) return rc;
  int n_qt = (max_new + FT_BQ - 1) / FT_BQ;
  long long n_items = (long long)H * n_qt * B;
  if (n_items > 0x7fffffffLL) return SLLM_ERR_ARG;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
  }
  if (hd == 64) {
    FtArgs a{(bf16*)out, seq_start, seq_pos0, block_table, max_pages, H, G, window, scale, err, n_qt, B, (int)n_items, 0};
    dim3 grid((unsigned)(n_items < 2LL * sm_count ? n_items : 2LL * sm_count));     // two blocks per SM that stay
    return ft_launch<64, 3>(mq, mk, mv, a, grid, stream);
  }
  int pair_heads = ((H / G) % 2 == 0) ? 1 : 0;
  n_items = pair_heads ? (long long)(H / 2) * n_qt * B : (long long)H * ((n_qt + 1) / 2) * B;
  FtArgs a{(bf16*)out, seq_start, seq_pos0, block_table, max_pages, H, G, window, scale, err, n_qt, B, (int)n_items, pair_heads};
  dim3 grid((unsigned)(n_items < (long long)sm_count ? n_items : (long long)sm_count));       // one block per SM that stays
  return fp_launch<128, 4>(mq, mk, mv, a, grid, stream);
}

// Sampling on the device, one thread block per row of float logits.
//
// Follows the reference's samplers: greedy = first index of the maximum with strict '>'
// (float32_ops.go:812-822); temperature = softmax(logits/T) with max subtraction, then the first
// index whose running sum reaches the uniform draw, else the last (model.go:805-838); top_k = the
// k largest logits, softmax(top/T), the same draw (model.go:723-752); top_p = softmax(logits/T),
// the shortest descending prefix whose sum reaches p, renormalised, the same draw
// (model.go:754-799); repeat penalty = each distinct recent token once, positive logit divided,
// other multiplied (sampling.go:314-336). Sums and the softmax run in double, as the reference
// samples in float64. Where the reference leaves an order open (which of several equal logits
// the quick-select keeps; the order of the kept tokens when drawing), the lower token index goes
// first. The uniform draw comes from Philox4x32-10 keyed by the sequence's seed with the
// sequence's draw index as the counter, so a sequence samples the same tokens alone or in a batch.
#include "common.cuh"
#include "philox.cuh"

#define SAMPLE_THREADS 1024

struct SampleParams {
  int strategy;  // 0 greedy, 1 temperature, 2 top_k, 3 top_p
  float temperature;
  int top_k;
  float top_p;
  unsigned seed_lo, seed_hi, draw_lo, draw_hi;
};

__device__ __forceinline__ double philox_uniform(unsigned seed_lo, unsigned seed_hi, unsigned c0, unsigned c1) {
  Philox4 r = philox4x32_10(c0, c1, 0u, 0u, seed_lo, seed_hi);
  unsigned long long bits = (((unsigned long long)r.w[0] << 32) | r.w[1]) >> 11;
  return (double)bits * (1.0 / 9007199254740992.0);
}

// order-preserving map float -> unsigned
__device__ __forceinline__ unsigned orderable(float f) {
  unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide sum of doubles, result to all threads
__device__ double block_sum_d(double v, double* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum_d(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  double t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.0;
  return warp_sum_d(t);
}

// exclusive prefix over threads (in thread order) and the total
__device__ double block_scan_excl_d(double v, double* red, double* total) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  double inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    double t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) red[wid] = inc;
  __syncthreads();
  double wsum = (lane < nw) ? red[lane] : 0.0;
  double winc = wsum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    double t = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += t;
  }
  double wexcl = __shfl_sync(0xffffffffu, winc - wsum, wid);
  *total = __shfl_sync(0xffffffffu, winc, nw - 1);
  return wexcl + inc - v;
}

// The per-sequence state record, 8 int32 words per cache slot (csrc and cache/store.py agree on it):
// tokens held, tokens generated, last token, flags, sampling key (two words), draw counter (two words).
#define SEQ_STATE_WORDS 8
#define SEQ_POS 0
#define SEQ_GENERATED 1
#define SEQ_LAST_TOKEN 2
#define SEQ_FLAGS 3
#define SEQ_KEY 4
#define SEQ_COUNTER 6
#define SEQ_FLAG_FINISHED 1

struct SampleStateArgs {
  const int* options;    // [4]: strategy, temperature bits, top_k, top_p bits -- the same for every row
  int* state;            // [slots][SEQ_STATE_WORDS]
  const int* slots;      // [rows] the slot of each row's sequence
  const int* pos_after;  // [rows] tokens the sequence holds after the step that made these logits (may be null)
  const int* stop_ids;   // [n_stop]
  int n_stop;
};

// What the reference does after it has picked a token: count it, remember it, stop on a stop token
// (model_f32.go:661-667) -- here as an update of the sequence's record by the thread that wrote the token.
__device__ __forceinline__ void seq_state_update(const SampleStateArgs& sa, int row, int token) {
  int* rec = sa.state + (size_t)sa.slots[row] * SEQ_STATE_WORDS;
  if (sa.pos_after) rec[SEQ_POS] = sa.pos_after[row];
  rec[SEQ_GENERATED] += 1;
  rec[SEQ_LAST_TOKEN] = token;
  unsigned lo = (unsigned)rec[SEQ_COUNTER] + 1u;
  rec[SEQ_COUNTER] = (int)lo;
  if (lo == 0u) rec[SEQ_COUNTER + 1] += 1;
  bool stop = false;
  for (int i = 0; i < sa.n_stop; i++) stop |= (sa.stop_ids[i] == token);
  if (stop) rec[SEQ_FLAGS] |= SEQ_FLAG_FINISHED;
}

// STATE: the row's parameters come from the options record and from its sequence's state record
// (key and draw counter), which the kernel then advances; else from params[row] and nothing is updated.
template <bool STATE>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int ldl, int V, const SampleParams* __restrict__ params,
                   SampleStateArgs sa, int* __restrict__ out) {
  __shared__ double red[32];
  __shared__ float red_f[32];
  __shared__ int red_i[32];
  __shared__ int pick;
  int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const float* lg = logits + (size_t)row * ldl;
  SampleParams p;
  if (STATE) {
    const int* rec = sa.state + (size_t)sa.slots[row] * SEQ_STATE_WORDS;
    p.strategy = sa.options[0];
    p.temperature = __int_as_float(sa.options[1]);
    p.top_k = sa.options[2];
    p.top_p = __int_as_float(sa.options[3]);
    p.seed_lo = (unsigned)rec[SEQ_KEY]; p.seed_hi = (unsigned)rec[SEQ_KEY + 1];
    p.draw_lo = (unsigned)rec[SEQ_COUNTER]; p.draw_hi = (unsigned)rec[SEQ_COUNTER + 1];
    __syncthreads();                 // every thread has read the record before thread 0 advances it
  } else {
    p = params[row];
  }
  int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  int i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);

  // ---- maximum and its first index (threads stride over the row here: neighbouring lanes read
  // neighbouring logits, several loads in flight; the running sums below need index order instead)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
#pragma unroll 8
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    float v = lg[i];
    if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
  }
  if (lane == 0) { red_f[wid] = best; red_i[wid] = best_i; }
  __syncthreads();
  if (wid == 0) {
    best = red_f[lane]; best_i = red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
    }
    if (lane == 0) { red_f[0] = best; red_i[0] = best_i; }
  }
  __syncthreads();
  best = red_f[0];
  best_i = red_i[0];
  if (p.strategy == 0 || !(p.temperature > 0.f)) {
    if (tid == 0) {
      out[row] = best_i;
      if (STATE) seq_state_update(sa, row, best_i);
    }
    return;
  }
  __syncthreads();

  double T = (double)p.temperature;
  double mx = (double)best / T;

  // ---- which tokens are kept: key > thr, or key == thr and among the first `ties_kept` such
  unsigned thr = 0u;            // orderable bits; 0 keeps everything
  long long ties_kept = 0x7fffffffffffLL;
  bool by_exp = false;          // key is exp(z - mx) (top_p) rather than the logit (top_k)
  if (p.strategy == 2) {
    int k = p.top_k <= 0 ? 50 : p.top_k;
    if (k > V) k = V;
    unsigned prefix = 0u;
    for (int bit = 31; bit >= 0; bit--) {
      unsigned cand = prefix | (1u << bit);
      double cnt = 0.0;
      for (int i = i0; i < i1; i++) cnt += orderable(lg[i]) >= cand ? 1.0 : 0.0;
      cnt = block_sum_d(cnt, red);
      if (cnt >= (double)k) prefix = cand;
    }
    thr = prefix;
    double gt = 0.0;
    for (int i = i0; i < i1; i++) gt += orderable(lg[i]) > thr ? 1.0 : 0.0;
    gt = block_sum_d(gt, red);
    ties_kept = (long long)k - (long long)gt;
  } else if (p.strategy == 3) {
    by_exp = true;
    double tot = 0.0;
    for (int i = i0; i < i1; i++) tot += (double)(float)exp((double)lg[i] / T - mx);
    tot = block_sum_d(tot, red);
    double target = (double)p.top_p * tot;
    unsigned prefix = 0u;
    for (int bit = 30; bit >= 0; bit--) {                       // exp() is positive: sign bit stays clear
      unsigned cand = prefix | (1u << bit);
      double s = 0.0;
      for (int i = i0; i < i1; i++) {
        float e = (float)exp((double)lg[i] / T - mx);
        if (__float_as_uint(e) >= cand) s += (double)e;
      }
      s = block_sum_d(s, red);
      if (s >= target) prefix = cand;
    }
    thr = prefix;
    double sgt = 0.0;
    for (int i = i0; i < i1; i++) {
      float e = (float)exp((double)lg[i] / T - mx);
      if (__float_as_uint(e) > thr) sgt += (double)e;
    }
    sgt = block_sum_d(sgt, red);
    double tv = (double)__uint_as_float(thr);
    ties_kept = tv > 0.0 ? (long long)ceil((target - sgt) / tv) : 0x7fffffffffffLL;
    if (ties_kept < 1) ties_kept = 1;
  }

  // rank of each thread's first tie among all ties (index order)
  double my_ties = 0.0;
  if (p.strategy >= 2) {
    for (int i = i0; i < i1; i++) {
      unsigned key = by_exp ? __float_as_uint((float)exp((double)lg[i] / T - mx)) : orderable(lg[i]);
      my_ties += key == thr ? 1.0 : 0.0;
    }
  }
  double tie_total;
  double tie_rank = block_scan_excl_d(my_ties, red, &tie_total);

  // ---- weights of the kept tokens, running sums in index order, the draw
  double local = 0.0;
  {
    long long rank = (long long)tie_rank;
    for (int i = i0; i < i1; i++) {
      double z = (double)lg[i] / T - mx;
      bool keep = true;
      if (p.strategy >= 2) {
        unsigned key = by_exp ? __float_as_uint((float)exp(z)) : orderable(lg[i]);
        keep = key > thr || (key == thr && rank++ < ties_kept);
      }
      if (keep) local += exp(z);
    }
  }
  double total;
  double before = block_scan_excl_d(local, red, &total);
  double u = philox_uniform(p.seed_lo, p.seed_hi, p.draw_lo, p.draw_hi);
  double inv = 1.0 / total;
  if (tid == 0) pick = 0x7fffffff;
  __syncthreads();
  {
    long long rank = (long long)tie_rank;
    double cum = before;
    int last_kept = -1;
    for (int i = i0; i < i1; i++) {
      double z = (double)lg[i] / T - mx;
      bool keep = true;
      if (p.strategy >= 2) {
        unsigned key = by_exp ? __float_as_uint((float)exp(z)) : orderable(lg[i]);
        keep = key > thr || (key == thr && rank++ < ties_kept);
      }
      if (!keep) continue;
      last_kept = i;
      cum += exp(z);
      if (u <= cum * inv) { atomicMin(&pick, i); break; }
    }
    __syncthreads();
    if (pick == 0x7fffffff) {                                   // rounding left the sum short: last kept token
      __syncthreads();
      if (tid == 0) pick = -1;
      __syncthreads();
      if (last_kept >= 0) atomicMax(&pick, last_kept);
      __syncthreads();
    }
  }
  if (tid == 0) {
    out[row] = pick;
    if (STATE) seq_state_update(sa, row, pick);
  }
}

// logits[row, t] /= penalty if positive else *= penalty, once for each distinct in-range token
// among the last `last_n` of recent[row, 0:count[row]].
__global__ void repeat_penalty_kernel(float* __restrict__ logits, int ldl, int V, const int* __restrict__ recent,
                                      int recent_ld, const int* __restrict__ counts, const float* __restrict__ penalty,
                                      int last_n) {
  int row = blockIdx.x;
  float pen = penalty[row];
  if (!(pen > 0.f)) return;
  int n = counts[row];
  int start = max(0, n - last_n);
  const int* r = recent + (size_t)row * recent_ld;
  for (int j = start + threadIdx.x; j < n; j += blockDim.x) {
    int t = r[j];
    if (t < 0 || t >= V) continue;
    bool dup = false;
    for (int e = start; e < j; e++) dup |= (r[e] == t);
    if (dup) continue;
    float* l = logits + (size_t)row * ldl + t;
    float v = *l;
    *l = v > 0.f ? v / pen : v * pen;
  }
}

SLLM_EXPORT int sllm_sample_rows(const float* logits, int ldl, int n_rows, int V, const void* params, int* out,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return SLLM_ERR_ARG;
  sample_rows_kernel<false><<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ldl, V, (const SampleParams*)params,
                                                                     SampleStateArgs{}, out);
  SLLM_RETURN_LAST();
}

// The same with every row's key and draw counter taken from its sequence's state record
// (state[slots[row]]), which is advanced: generated count, last token, counter, finished flag when
// the token is one of stop_ids, and the position if pos_after is given. `options`: 4 int32 on the
// device (strategy, temperature bits, top_k, top_p bits). Nothing comes from the host per call.
SLLM_EXPORT int sllm_sample_rows_state(const float* logits, int ldl, int n_rows, int V, const int* options, int* state,
                                       const int* slots, const int* pos_after, const int* stop_ids, int n_stop, int* out,
                                       cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0 || n_stop < 0 || !options || !state || !slots) return SLLM_ERR_ARG;
  SampleStateArgs sa{options, state, slots, pos_after, stop_ids, n_stop};
  sample_rows_kernel<true><<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ldl, V, nullptr, sa, out);
  SLLM_RETURN_LAST();
}

SLLM_EXPORT int sllm_repeat_penalty(float* logits, int ldl, int n_rows, int V, const int* recent, int recent_ld,
                                    const int* counts, const float* penalty, int last_n, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  repeat_penalty_kernel<<<n_rows, 128, 0, stream>>>(logits, ldl, V, recent, recent_ld, counts, penalty, last_n);
  SLLM_RETURN_LAST();
}

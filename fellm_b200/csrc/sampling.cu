// Sampling on the device: greedy, temperature, top-k, min-p, top-p, repetition / frequency /
// presence penalties and logit bias, one thread block per row of logits.
//
// FeLLM samples on the host (crates/fellm-runtime/src/sampling.rs:325-394): adjust logits
// (repetition, frequency, presence, bias: 554-586) -> / temperature -> keep the k best (ties:
// lower id, 26-33) -> softmax over them -> drop p < min_p * p_max, renormalise -> shortest prefix
// by descending p whose mass reaches top_p, renormalise -> order by token id -> inverse-CDF draw
// with one uniform number; greedy (temperature <= 0 or top_k == 1) is argmax of the adjusted
// logits, ties to the lower id (588-604; device argmax_token, oxide_kernels.rs:116-160).
// The same steps run here without sorting: every filter keeps a prefix of the order (value
// descending, id ascending), so it is a *cut* (kt, q): all tokens whose key is above kt, plus the
// q lowest ids whose key equals kt.  Cuts are found by an 8-bit radix descent over the 32-bit
// order-preserving key of the value, weighting tokens by 1 (top-k) or by their probability in
// 2^-40 fixed point (top-p); integer weights make every sum exact, hence reproducible.
// The uniform number comes from splitmix64(seed + draw index) (FeLLM seeds ChaCha8 with that
// value, 384-393,606-612; the streams differ, the seeding rule is the same).
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define FIX_ONE 1099511627776.0f     // 2^40

typedef unsigned long long u64;

struct RowParams {
  float temperature, top_p, min_p, rep_pen, freq_pen, pres_pen;
  int top_k, slot, bias_begin, bias_end;
  u64 seed;
};

struct Row {
  const float* logits;
  const int* counts;       // [V] of this row's request, or null
  const int* bias_tok;
  const float* bias_val;
  int bias_begin, bias_end;
  float rep_pen, freq_pen, pres_pen, inv_temp;
  int V;
  // sampling.rs:554-586
  __device__ __forceinline__ float adjusted(int v) const {
    float x = logits[v];
    int c = counts ? counts[v] : 0;
    if (c > 0) {
      if (rep_pen > 1.0f && isfinite(rep_pen)) x = x < 0.f ? x * rep_pen : x / rep_pen;
      x = x - freq_pen * (float)c - pres_pen;
    }
    for (int i = bias_begin; i < bias_end; ++i)
      if (bias_tok[i] == v) x += bias_val[i];
    return x;
  }
  __device__ __forceinline__ float val(int v) const { return adjusted(v) * inv_temp; }
};

__device__ __forceinline__ unsigned key_of(float x) {
  if (x != x) return 0u;                               // NaN sorts last
  unsigned b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float val_of(unsigned k) {
  unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

__device__ float block_max(float v, float* sm) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < SAMPLE_THREADS / 32 ? sm[threadIdx.x] : -INFINITY;
    t = warp_max(t);
    if (threadIdx.x == 0) sm[0] = t;
  }
  __syncthreads();
  float r = sm[0];
  __syncthreads();
  return r;
}
__device__ float block_sum(float v, float* sm) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < SAMPLE_THREADS / 32 ? sm[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) sm[0] = t;
  }
  __syncthreads();
  float r = sm[0];
  __syncthreads();
  return r;
}
__device__ __forceinline__ u64 shfl_up_u64(u64 v, int d) {
  unsigned lo = __shfl_up_sync(0xffffffffu, (unsigned)v, d), hi = __shfl_up_sync(0xffffffffu, (unsigned)(v >> 32), d);
  return ((u64)hi << 32) | lo;
}
// inclusive scan over the block in thread order; *total = the block's sum
__device__ u64 block_scan_incl(u64 v, u64* sm, u64* total) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) { u64 t = shfl_up_u64(v, d); if (lane >= d) v += t; }
  if (lane == 31) sm[w] = v;
  __syncthreads();
  if (w == 0) {
    u64 t = lane < SAMPLE_THREADS / 32 ? sm[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { u64 u = shfl_up_u64(t, d); if (lane >= d) t += u; }
    sm[lane] = t;
  }
  __syncthreads();
  u64 off = w ? sm[w - 1] : 0;
  *total = sm[SAMPLE_THREADS / 32 - 1];
  __syncthreads();
  return v + off;
}

// A cut keeps every token with key > kt and the q lowest ids with key == kt.
struct Cut { unsigned kt; u64 q; };

struct Shared {
  u64 hist[8][256];            // one histogram per 4 warps: fewer same-address collisions
  u64 scan[32];
  float red[32];
  unsigned prefix; int found; u64 remaining; u64 bin_total;
  int pick, last;
};

// Weight of a token for the descent: MODE 0 -> 1 (top-k); MODE 1 -> probability in fixed point.
struct Weigher {
  int mode; float m, sum1, sum2; bool use_sum2;
  __device__ __forceinline__ float prob(float val) const {
    float p = expf(val - m) / sum1;
    return use_sum2 ? p / sum2 : p;
  }
  __device__ __forceinline__ u64 w(float val) const {
    return mode == 0 ? 1ull : __float2ull_rd(prob(val) * FIX_ONE);
  }
};

// Finds the cut whose kept weight first reaches `target`, among tokens inside `outer` whose
// probability passes minp_thr.  If all of them together stay below target, returns `outer`.
__device__ Cut radix_cut(const Row& r, Shared* s, u64 target, const Weigher& wg, Cut outer,
                         float minp_thr, const Weigher& pg) {
  int warp = (threadIdx.x >> 5) & 7;
  if (threadIdx.x == 0) { s->prefix = 0; s->remaining = target; s->found = 1; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 8 * 256; i += SAMPLE_THREADS) (&s->hist[0][0])[i] = 0;
    __syncthreads();
    unsigned prefix = s->prefix;
    for (int v = threadIdx.x; v < r.V; v += SAMPLE_THREADS) {
      float x = r.val(v);
      unsigned k = key_of(x);
      if (k <= outer.kt) continue;                      // ties of the outer cut are added below
      if (minp_thr > 0.f && pg.prob(x) < minp_thr) continue;
      if (pass > 0 && (k >> (shift + 8)) != (prefix >> (shift + 8))) continue;
      atomicAdd(&s->hist[warp][(k >> shift) & 255], wg.w(x));
    }
    if (threadIdx.x == 0 && outer.q > 0) {
      unsigned k = outer.kt;
      float x = val_of(k);
      bool ok = !(minp_thr > 0.f && pg.prob(x) < minp_thr);
      if (ok && (pass == 0 || (k >> (shift + 8)) == (prefix >> (shift + 8))))
        atomicAdd(&s->hist[warp][(k >> shift) & 255], outer.q * wg.w(x));
    }
    __syncthreads();
    if (threadIdx.x < 256) {                            // fold the per-warp histograms
      u64 t = 0;
      for (int w = 0; w < 8; ++w) t += s->hist[w][threadIdx.x];
      s->hist[0][threadIdx.x] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      u64 cum = 0, rem = s->remaining;
      int d = 255;
      for (; d >= 0; --d) {
        u64 h = s->hist[0][d];
        if (cum + h >= rem) break;
        cum += h;
      }
      if (d < 0) s->found = 0;
      else { s->remaining = rem - cum; s->prefix = prefix | ((unsigned)d << shift); s->bin_total = s->hist[0][d]; }
    }
    __syncthreads();
    if (!s->found) return outer;
  }
  Cut c;
  c.kt = s->prefix;
  u64 wt = wg.w(val_of(c.kt));
  if (wt == 0) wt = 1;
  u64 n_ties = s->bin_total / wt;
  c.q = (s->remaining + wt - 1) / wt;
  if (c.q > n_ties) c.q = n_ties;
  if (c.kt == outer.kt && c.q > outer.q) c.q = outer.q;
  __syncthreads();
  return c;
}

__device__ __forceinline__ u64 splitmix64(u64 x) {
  x += 0x9E3779B97F4A7C15ull;
  u64 z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const RowParams* __restrict__ params,
              int* __restrict__ counts, const int* __restrict__ bias_tok, const float* __restrict__ bias_val,
              int* __restrict__ out_tokens, float* __restrict__ out_probs, int update_counts) {
  FELLM_TRACE_SCOPE(TRACE_SAMPLE);
  __shared__ Shared s;
  int row = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  RowParams p = params[row];
  Row r;
  r.logits = logits + (size_t)row * V;
  bool pen = counts && ((p.rep_pen > 1.0f && isfinite(p.rep_pen)) || p.freq_pen != 0.f || p.pres_pen != 0.f);
  int* my_counts = counts ? counts + (size_t)p.slot * V : nullptr;
  r.counts = pen ? my_counts : nullptr;
  r.bias_tok = bias_tok; r.bias_val = bias_val; r.bias_begin = p.bias_begin; r.bias_end = p.bias_end;
  r.rep_pen = p.rep_pen; r.freq_pen = p.freq_pen; r.pres_pen = p.pres_pen; r.V = V;
  float* probs = out_probs ? out_probs + (size_t)row * V : nullptr;

  bool greedy = p.temperature <= 0.f || p.top_k == 1;
  if (greedy) {
    // argmax of the adjusted logits, first maximum wins (sampling.rs:588-604)
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) {
      float x = r.adjusted(v);
      if (x > best) { best = x; bi = v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    __shared__ float gb[32]; __shared__ int gi[32];
    if ((threadIdx.x & 31) == 0) { gb[threadIdx.x >> 5] = best; gi[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
      best = gb[threadIdx.x]; bi = gi[threadIdx.x];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (threadIdx.x == 0) {
        if (bi == 0x7fffffff) bi = 0;                   // all -inf / NaN: token 0, as the reference's loop
        out_tokens[row] = bi;
        if (update_counts && my_counts) my_counts[bi] += 1;
      }
    }
    if (probs) {
      __syncthreads();
      int tok = out_tokens[row];
      for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) probs[v] = v == tok ? 1.f : 0.f;
    }
    return;
  }

  r.inv_temp = 1.0f / fmaxf(p.temperature, 1.1920929e-07f);
  // top-k cut
  Cut all; all.kt = 0u; all.q = 0;                       // key 0 is NaN only: everything is above it
  Weigher unit; unit.mode = 0; unit.m = 0; unit.sum1 = 1; unit.sum2 = 1; unit.use_sum2 = false;
  Cut cut = all;
  if (p.top_k > 0 && p.top_k < V) cut = radix_cut(r, &s, (u64)p.top_k, unit, all, 0.f, unit);

  // softmax over the kept tokens
  float m = -INFINITY;
  for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) {
    float x = r.val(v);
    if (key_of(x) >= cut.kt && key_of(x) > 0u) m = fmaxf(m, x);
  }
  m = block_max(m, s.red);
  float part = 0.f;
  for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) {
    float x = r.val(v);
    if (key_of(x) > cut.kt) part += expf(x - m);
  }
  float sum1 = block_sum(part, s.red) + (cut.q ? (float)cut.q * expf(val_of(cut.kt) - m) : 0.f);
  Weigher pg; pg.mode = 1; pg.m = m; pg.sum1 = sum1; pg.sum2 = 1.f; pg.use_sum2 = false;

  // min-p: drop p < p_max * min_p, renormalise
  float minp_thr = 0.f;
  if (p.min_p > 0.f && p.min_p < 1.f) {
    minp_thr = pg.prob(m) * p.min_p;
    part = 0.f;
    for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) {
      float x = r.val(v);
      if (key_of(x) > cut.kt) { float q = pg.prob(x); if (q >= minp_thr) part += q; }
    }
    float tq = cut.q ? pg.prob(val_of(cut.kt)) : 0.f;
    float sum2 = block_sum(part, s.red) + ((cut.q && tq >= minp_thr) ? (float)cut.q * tq : 0.f);
    if (sum2 > 0.f) { pg.sum2 = sum2; pg.use_sum2 = true; }
  }
  Weigher base = pg;                                     // p before the min-p renormalisation:
  base.use_sum2 = false;                                 // what the min-p threshold is compared with

  // top-p cut: shortest prefix whose mass reaches top_p
  float sum3 = 1.f; bool use_sum3 = false;
  if (p.top_p < 1.f && p.top_p > 0.f) {
    cut = radix_cut(r, &s, __float2ull_ru(p.top_p * FIX_ONE), pg, cut, minp_thr, base);
    part = 0.f;
    for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) {
      float x = r.val(v);
      if (key_of(x) > cut.kt) { float q = pg.prob(x); if (!(minp_thr > 0.f && base.prob(x) < minp_thr)) part += q; }
    }
    float tq = cut.q ? pg.prob(val_of(cut.kt)) : 0.f;
    bool tie_ok = cut.q && !(minp_thr > 0.f && base.prob(val_of(cut.kt)) < minp_thr);
    sum3 = block_sum(part, s.red) + (tie_ok ? (float)cut.q * tq : 0.f);
    use_sum3 = sum3 > 0.f;
  }

  // draw in token-id order
  u64 bits = splitmix64(p.seed);
  float u = (float)(bits >> 40) * (1.0f / 16777216.0f);
  u64 target = __float2ull_rd(u * FIX_ONE);
  if (threadIdx.x == 0) { s.pick = 0x7fffffff; s.last = -1; }
  __syncthreads();
  u64 tie_run = 0, w_run = 0;
  for (int base_v = 0; base_v < V; base_v += SAMPLE_THREADS) {
    int v = base_v + threadIdx.x;
    float x = 0.f; unsigned k = 0; bool ok = false;
    if (v < V) {
      x = r.val(v); k = key_of(x);
      ok = k > 0u && k >= cut.kt && !(minp_thr > 0.f && base.prob(x) < minp_thr);
    }
    u64 tt;
    u64 tie_rank = block_scan_incl((ok && k == cut.kt) ? 1ull : 0ull, s.scan, &tt);
    bool member = ok && (k > cut.kt || (tie_run + tie_rank - 1) < cut.q);
    float pf = 0.f;
    if (member) { pf = pg.prob(x); if (use_sum3) pf = pf / sum3; }
    if (probs && v < V) probs[v] = pf;
    u64 wt = member ? __float2ull_rd(pf * FIX_ONE) : 0ull;
    u64 wtot;
    u64 cum = w_run + block_scan_incl(wt, s.scan, &wtot);
    if (member) {
      if (cum > target) atomicMin(&s.pick, v);
      atomicMax(&s.last, v);
    }
    tie_run += tt; w_run += wtot;
    __syncthreads();
    if (s.pick != 0x7fffffff && !probs) break;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tok = s.pick != 0x7fffffff ? s.pick : (s.last >= 0 ? s.last : 0);
    out_tokens[row] = tok;
    if (update_counts && my_counts) my_counts[tok] += 1;
  }
}

// counts[slot, token] += 1 for a list of (slot, token): primes a request's history with its prompt.
__global__ void count_tokens_kernel(int* __restrict__ counts, int V, const int* __restrict__ slots,
                                    const int* __restrict__ tokens, int n) {
  FELLM_TRACE_SCOPE(TRACE_COUNT_TOKENS);
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && tokens[i] >= 0 && tokens[i] < V) atomicAdd(&counts[(size_t)slots[i] * V + tokens[i]], 1);
}

FELLM_API int fellm_sample(const float* logits, int rows, int V, const void* params, int* counts,
                           const int* bias_tok, const float* bias_val, int* out_tokens, float* out_probs,
                           int update_counts, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!logits || !params || !out_tokens || V < 1) return FELLM_ERR_ARG;
  return launch_k(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, 1, logits, V, (const RowParams*)params,
                  counts, bias_tok, bias_val, out_tokens, out_probs, update_counts);
}

FELLM_API int fellm_count_tokens(int* counts, int V, const int* slots, const int* tokens, int n,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  count_tokens_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(counts, V, slots, tokens, n);
  return launch_status();
}

// ---- greedy fast path: rows without penalties or bias.  Two launches: every row is cut into
// ARGMAX_CHUNKS pieces reduced by one block each, then one warp per row reduces the pieces.
// Ties go to the lower id at both stages (sampling.rs:588-604).
#define ARGMAX_CHUNKS 64
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int V, float* __restrict__ pval, int* __restrict__ pidx) {
  FELLM_TRACE_SCOPE(TRACE_ARGMAX_PARTIAL);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  int row = blockIdx.y, chunk = blockIdx.x;
  int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
  int lo = chunk * per, hi = min(V, lo + per);
  const float* lg = logits + (size_t)row * V;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int v = lo + threadIdx.x; v < hi; v += 256) {
    float x = lg[v];
    if (x > best) { best = x; bi = v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  __shared__ float sb[8]; __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sb[w] > best || (sb[w] == best && si[w] < bi)) { best = sb[w]; bi = si[w]; }
    pval[row * ARGMAX_CHUNKS + chunk] = best;
    pidx[row * ARGMAX_CHUNKS + chunk] = bi;
  }
}
__global__ void __launch_bounds__(32)
argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int* __restrict__ out_tokens) {
  FELLM_TRACE_SCOPE(TRACE_ARGMAX_FINAL);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  int row = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int c = lane; c < ARGMAX_CHUNKS; c += 32) {
    float x = pval[row * ARGMAX_CHUNKS + c]; int i = pidx[row * ARGMAX_CHUNKS + c];
    if (x > best || (x == best && i < bi)) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  if (lane == 0) out_tokens[row] = bi == 0x7fffffff ? 0 : bi;
}

// pval / pidx: scratch of rows * 64 entries each.
FELLM_API int fellm_argmax_rows(const float* logits, int rows, int V, float* pval, int* pidx, int* out_tokens,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!logits || !pval || !pidx || !out_tokens || V < 1) return FELLM_ERR_ARG;
  int e = launch_k(argmax_partial_kernel, dim3(ARGMAX_CHUNKS, rows), dim3(256), 0, stream, 1, logits, V, pval, pidx);
  if (e) return e;
  return launch_k(argmax_final_kernel, dim3(rows), dim3(32), 0, stream, 1, (const float*)pval, (const int*)pidx, out_tokens);
}

FELLM_API int fellm_sample_params_size() { return (int)sizeof(RowParams); }

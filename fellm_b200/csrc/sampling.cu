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

// ------------------------------------------------------------------------------------------------
// The same sampler with a CLUSTER of eight CTAs per row.  One block per row leaves a row of 65,536
// logits to one SM: a dozen passes over the row cost 0.35 ms, as much as the whole decode step
// before it.  Here every CTA keeps an eighth of the row in shared memory (penalties, bias and
// temperature applied once), histograms and sums are combined over the cluster through
// distributed shared memory in rank order (so every CTA computes the same numbers, and the same
// numbers every run), and the draw walks only the one warp that holds the target.
// Same cuts, same tie rule (lower id first), same fixed-point weights as sample_kernel above.
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SC_CL 8
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)

struct CShared {
  u64 hist[2][256];              // this CTA's histogram of the pass, two in turn
  u64 ghist[256];                // the cluster's
  float xf[2]; float xf2[2][2]; u64 xu[2][2]; int xi[2];          // this CTA's share of a cluster-wide reduction, two in turn
  float wf[SC_WARPS]; u64 wu[SC_WARPS][2]; int wi[SC_WARPS];
  u64 warp_ties[SC_WARPS], warp_w[SC_WARPS];
  unsigned prefix; int found; u64 remaining, bin_total;
  float bf, bf2; u64 bu[2]; int bi;
};

struct ClCtx {
  CShared* s; int pp; int rank;
};

__device__ __forceinline__ u64 shfl_down_u64(u64 v, int d) {
  unsigned lo = __shfl_down_sync(0xffffffffu, (unsigned)v, d), hi = __shfl_down_sync(0xffffffffu, (unsigned)(v >> 32), d);
  return ((u64)hi << 32) | lo;
}
__device__ __forceinline__ u64 shfl_xor_u64(u64 v, int d) {
  unsigned lo = __shfl_xor_sync(0xffffffffu, (unsigned)v, d), hi = __shfl_xor_sync(0xffffffffu, (unsigned)(v >> 32), d);
  return ((u64)hi << 32) | lo;
}
__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += shfl_xor_u64(v, o);
  return v;
}

// Cluster-wide maximum / ordered sum / minimum: every thread of every CTA of the cluster calls these.
__device__ float cl_max(ClCtx& c, float v) {
  CShared* s = c.s;
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) s->wf[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = -INFINITY;
    for (int w = 0; w < SC_WARPS; ++w) t = fmaxf(t, s->wf[w]);
    s->xf[c.pp] = t;
  }
  cg::this_cluster().sync();
  if (threadIdx.x == 0) {
    float t = -INFINITY;
    for (int r = 0; r < SC_CL; ++r) t = fmaxf(t, *cg::this_cluster().map_shared_rank(&s->xf[c.pp], r));
    s->bf = t;
  }
  __syncthreads();
  c.pp ^= 1;
  return s->bf;
}
__device__ float cl_sum(ClCtx& c, float v) {
  CShared* s = c.s;
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) s->wf[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < SC_WARPS; ++w) t += s->wf[w];
    s->xf[c.pp] = t;
  }
  cg::this_cluster().sync();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int r = 0; r < SC_CL; ++r) t += *cg::this_cluster().map_shared_rank(&s->xf[c.pp], r);
    s->bf = t;
  }
  __syncthreads();
  c.pp ^= 1;
  return s->bf;
}
__device__ int cl_min_int(ClCtx& c, int v) {
  CShared* s = c.s;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) s->wi[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0x7fffffff;
    for (int w = 0; w < SC_WARPS; ++w) t = min(t, s->wi[w]);
    s->xi[c.pp] = t;
  }
  cg::this_cluster().sync();
  if (threadIdx.x == 0) {
    int t = 0x7fffffff;
    for (int r = 0; r < SC_CL; ++r) t = min(t, *cg::this_cluster().map_shared_rank(&s->xi[c.pp], r));
    s->bi = t;
  }
  __syncthreads();
  c.pp ^= 1;
  return s->bi;
}
// Per-warp u64 values (already in s->warp_ties / s->warp_w style arrays `mine`): returns the sum of
// all warps of the CTAs before this one (*before) and of the whole cluster (*total).
__device__ void cl_prefix_u64(ClCtx& c, const u64* mine, u64* before, u64* total) {
  CShared* s = c.s;
  __syncthreads();
  if (threadIdx.x == 0) {
    u64 t = 0;
    for (int w = 0; w < SC_WARPS; ++w) t += mine[w];
    s->xu[c.pp][0] = t;
  }
  cg::this_cluster().sync();
  if (threadIdx.x == 0) {
    u64 b = 0, t = 0;
    for (int r = 0; r < SC_CL; ++r) {
      u64 x = *cg::this_cluster().map_shared_rank(&s->xu[c.pp][0], r);
      if (r < c.rank) b += x;
      t += x;
    }
    s->bu[0] = b; s->bu[1] = t;
  }
  __syncthreads();
  c.pp ^= 1;
  *before = s->bu[0]; *total = s->bu[1];
}

// One histogram entry from every lane of a warp (all 32 call it).  When the whole warp hits one bin
// (the top bytes of a row of logits are nearly all the same) one lane adds the warp's sum.
__device__ __forceinline__ void hist_add(u64* hist, unsigned bin, u64 w, bool active, bool unit) {
  const unsigned am = __ballot_sync(0xffffffffu, active);
  if (unit) {
    // weights of 1 (top-k): the lanes of a bin are counted by one of them (a row of logits has two or
    // three distinct top bytes: 32 atomics on as many addresses would take turns)
    if (active) {
      const unsigned peers = __match_any_sync(am, bin);
      if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (u64)__popc(peers));
    }
    return;
  }
  if (__popc(am) < 8) {                                  // few lanes: they take their turns
    if (active) atomicAdd(&hist[bin], w);
    return;
  }
  // probability weights (top-p), many lanes: bin by bin (a row has few distinct ones), the warp sums
  // the bin's weights and one lane adds them
  unsigned left = am;
  while (left) {
    const int src = __ffs(left) - 1;
    const unsigned b = __shfl_sync(0xffffffffu, bin, src);
    const bool mine = active && bin == b;
    const unsigned grp = __ballot_sync(0xffffffffu, mine);
    const u64 t = warp_sum_u64(mine ? w : 0ull);
    if ((int)(threadIdx.x & 31) == src) atomicAdd(&hist[b], t);
    left &= ~grp;
  }
}

// The cut whose kept weight first reaches `target` (see radix_cut), over the cluster's row.
// vals: this CTA's slice in shared memory (n_local of them); the warp walks [w0, w1).
__device__ Cut radix_cut_cl(ClCtx& c, const float* vals, int w0, int w1, u64 target, const Weigher& wg, Cut outer,
                            float minp_thr, const Weigher& pg) {
  CShared* s = c.s;
  const int lane = threadIdx.x & 31;
  unsigned prefix = 0;
  u64 remaining = target, bin_total = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    u64* hist = s->hist[c.pp];
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      bool active = i < w1;
      float x = active ? vals[i] : 0.f;
      unsigned k = key_of(x);
      active = active && k > outer.kt && !(minp_thr > 0.f && pg.prob(x) < minp_thr) &&
               (pass == 0 || (k >> (shift + 8)) == (prefix >> (shift + 8)));
      hist_add(hist, (k >> shift) & 255, active ? wg.w(x) : 0ull, active, wg.mode == 0);
    }
    if (c.rank == 0 && threadIdx.x == 0 && outer.q > 0) {          // the ties of the outer cut, once
      unsigned k = outer.kt;
      float x = val_of(k);
      bool ok = !(minp_thr > 0.f && pg.prob(x) < minp_thr);
      if (ok && (pass == 0 || (k >> (shift + 8)) == (prefix >> (shift + 8)))) atomicAdd(&hist[(k >> shift) & 255], outer.q * wg.w(x));
    }
    __syncthreads();
    cg::this_cluster().sync();
    if (threadIdx.x < 256) {
      u64 t = 0;
      for (int r = 0; r < SC_CL; ++r) t += *cg::this_cluster().map_shared_rank(&hist[threadIdx.x], r);
      s->ghist[threadIdx.x] = t;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // lane l holds bins 8l .. 8l+7; from the top bin down, the first bin at which the running sum reaches `remaining`
      u64 tl = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) tl += s->ghist[8 * lane + j];
      u64 incl = tl;                                               // sum over lanes >= this one
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) { u64 t = shfl_down_u64(incl, d); if (lane + d < 32) incl += t; }
      const unsigned crossing = __ballot_sync(0xffffffffu, incl >= remaining);
      if (crossing == 0) {
        if (lane == 0) s->found = 0;
      } else {
        const int l = 31 - __clz(crossing);
        if (lane == l) {
          u64 cum = incl - tl;
          int d = 8 * lane + 7;
          for (; d > 8 * lane; --d) {
            u64 h = s->ghist[d];
            if (cum + h >= remaining) break;
            cum += h;
          }
          s->found = 1; s->remaining = remaining - cum; s->prefix = prefix | ((unsigned)d << shift); s->bin_total = s->ghist[d];
        }
      }
    }
    __syncthreads();
    const int found = s->found;
    if (found) { remaining = s->remaining; prefix = s->prefix; bin_total = s->bin_total; }
    c.pp ^= 1;
    __syncthreads();
    if (!found) return outer;
  }
  Cut cut;
  cut.kt = prefix;
  u64 wt = wg.w(val_of(cut.kt));
  if (wt == 0) wt = 1;
  u64 n_ties = bin_total / wt;
  cut.q = (remaining + wt - 1) / wt;
  if (cut.q > n_ties) cut.q = n_ties;
  if (cut.kt == outer.kt && cut.q > outer.q) cut.q = outer.q;
  return cut;
}

__global__ void __cluster_dims__(SC_CL, 1, 1) __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int V, int slice, const RowParams* __restrict__ params,
                      int* __restrict__ counts, const int* __restrict__ bias_tok, const float* __restrict__ bias_val,
                      int* __restrict__ out_tokens, float* __restrict__ out_probs, int update_counts) {
  FELLM_TRACE_SCOPE(TRACE_SAMPLE);
  extern __shared__ __align__(16) float vals[];          // this CTA's slice: adjusted logits (/ temperature)
  __shared__ CShared s;
  ClCtx c; c.s = &s; c.pp = 0; c.rank = (int)cg::this_cluster().block_rank();
  const int row = blockIdx.x / SC_CL;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  const RowParams p = params[row];
  Row r;
  r.logits = logits + (size_t)row * V;
  const bool pen = counts && ((p.rep_pen > 1.0f && isfinite(p.rep_pen)) || p.freq_pen != 0.f || p.pres_pen != 0.f);
  int* my_counts = counts ? counts + (size_t)p.slot * V : nullptr;
  r.counts = pen ? my_counts : nullptr;
  r.bias_tok = bias_tok; r.bias_val = bias_val; r.bias_begin = p.bias_begin; r.bias_end = p.bias_end;
  r.rep_pen = p.rep_pen; r.freq_pen = p.freq_pen; r.pres_pen = p.pres_pen; r.V = V;
  float* probs = out_probs ? out_probs + (size_t)row * V : nullptr;
  const bool greedy = p.temperature <= 0.f || p.top_k == 1;
  r.inv_temp = greedy ? 1.0f : 1.0f / fmaxf(p.temperature, 1.1920929e-07f);

  // ids of this CTA: [v0, v0 + n_local); warp w walks the local range [w0, w1), lane-strided
  const int v0 = c.rank * slice, n_local = max(0, min(V, v0 + slice) - v0);
  for (int i = threadIdx.x; i < n_local; i += SC_THREADS) vals[i] = r.adjusted(v0 + i) * r.inv_temp;
  __syncthreads();
  const int per_warp = (slice + SC_WARPS - 1) / SC_WARPS;
  const int w0 = min(n_local, warp * per_warp), w1 = min(n_local, w0 + per_warp);

  if (greedy) {
    // first maximum of the adjusted logits (sampling.rs:588-604)
    float best = -INFINITY;
    for (int i = w0 + lane; i < w1; i += 32) best = fmaxf(best, vals[i]);
    const float m = cl_max(c, best);
    int bi = 0x7fffffff;
    for (int i = w0 + lane; i < w1; i += 32) if (vals[i] == m) bi = min(bi, v0 + i);
    int tok = cl_min_int(c, bi);
    if (!(m > -INFINITY) || tok == 0x7fffffff) tok = 0;  // all -inf / NaN: token 0, as the reference's loop
    if (c.rank == 0 && threadIdx.x == 0) {
      out_tokens[row] = tok;
      if (update_counts && my_counts) my_counts[tok] += 1;
    }
    if (probs) for (int i = threadIdx.x; i < n_local; i += SC_THREADS) probs[v0 + i] = (v0 + i) == tok ? 1.f : 0.f;
    cg::this_cluster().sync();                           // nobody leaves while its shared memory may be read
    return;
  }

  // top-k cut
  Cut all; all.kt = 0u; all.q = 0;                       // key 0 is NaN only: everything is above it
  Weigher unit; unit.mode = 0; unit.m = 0; unit.sum1 = 1; unit.sum2 = 1; unit.use_sum2 = false;
  Cut cut = all;
  if (p.top_k > 0 && p.top_k < V) cut = radix_cut_cl(c, vals, w0, w1, (u64)p.top_k, unit, all, 0.f, unit);

  // softmax over the kept tokens: every CTA's maximum and its sum relative to it go round in one
  // exchange; the cluster's maximum and sum follow in rank order
  float part = -INFINITY;
  for (int i = w0 + lane; i < w1; i += 32) { float x = vals[i]; unsigned k = key_of(x); if (k >= cut.kt && k > 0u) part = fmaxf(part, x); }
  float m, sum1;
  {
    part = warp_max(part);
    if (lane == 0) s.wf[warp] = part;
    __syncthreads();
    float m_cta = -INFINITY;
    for (int w = 0; w < SC_WARPS; ++w) m_cta = fmaxf(m_cta, s.wf[w]);
    __syncthreads();
    float ps = 0.f;
    for (int i = w0 + lane; i < w1; i += 32) { float x = vals[i]; if (key_of(x) > cut.kt) ps += expf(x - m_cta); }
    ps = warp_sum(ps);
    if (lane == 0) s.wf[warp] = ps;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < SC_WARPS; ++w) t += s.wf[w];
      s.xf2[c.pp][0] = m_cta; s.xf2[c.pp][1] = t;
    }
    cg::this_cluster().sync();
    if (threadIdx.x == 0) {
      float mm = -INFINITY, ms[SC_CL], ss[SC_CL];
      for (int r = 0; r < SC_CL; ++r) {
        const float* q = cg::this_cluster().map_shared_rank(&s.xf2[c.pp][0], r);
        ms[r] = q[0]; ss[r] = q[1];
        mm = fmaxf(mm, ms[r]);
      }
      float t = 0.f;
      for (int r = 0; r < SC_CL; ++r) if (ss[r] != 0.f) t += ss[r] * expf(ms[r] - mm);
      s.bf = mm; s.bf2 = t;
    }
    __syncthreads();
    c.pp ^= 1;
    m = s.bf;
    sum1 = s.bf2 + (cut.q ? (float)cut.q * expf(val_of(cut.kt) - m) : 0.f);
  }
  Weigher pg; pg.mode = 1; pg.m = m; pg.sum1 = sum1; pg.sum2 = 1.f; pg.use_sum2 = false;

  // min-p: drop p < p_max * min_p, renormalise
  float minp_thr = 0.f;
  if (p.min_p > 0.f && p.min_p < 1.f) {
    minp_thr = pg.prob(m) * p.min_p;
    part = 0.f;
    for (int i = w0 + lane; i < w1; i += 32) {
      float x = vals[i];
      if (key_of(x) > cut.kt) { float q = pg.prob(x); if (q >= minp_thr) part += q; }
    }
    float tq = cut.q ? pg.prob(val_of(cut.kt)) : 0.f;
    float sum2 = cl_sum(c, part) + ((cut.q && tq >= minp_thr) ? (float)cut.q * tq : 0.f);
    if (sum2 > 0.f) { pg.sum2 = sum2; pg.use_sum2 = true; }
  }
  Weigher base = pg;                                     // p before the min-p renormalisation:
  base.use_sum2 = false;                                 // what the min-p threshold is compared with

  // top-p cut: shortest prefix whose mass reaches top_p
  float sum3 = 1.f; bool use_sum3 = false;
  if (p.top_p < 1.f && p.top_p > 0.f) {
    cut = radix_cut_cl(c, vals, w0, w1, __float2ull_ru(p.top_p * FIX_ONE), pg, cut, minp_thr, base);
    part = 0.f;
    for (int i = w0 + lane; i < w1; i += 32) {
      float x = vals[i];
      if (key_of(x) > cut.kt) { float q = pg.prob(x); if (!(minp_thr > 0.f && base.prob(x) < minp_thr)) part += q; }
    }
    float tq = cut.q ? pg.prob(val_of(cut.kt)) : 0.f;
    bool tie_ok = cut.q && !(minp_thr > 0.f && base.prob(val_of(cut.kt)) < minp_thr);
    sum3 = cl_sum(c, part) + (tie_ok ? (float)cut.q * tq : 0.f);
    use_sum3 = sum3 > 0.f;
  }

  // draw in token-id order.  Ties of the cut are kept lowest id first: their ranks come first.
  u64 bits = splitmix64(p.seed);
  float u = (float)(bits >> 40) * (1.0f / 16777216.0f);
  const u64 target = __float2ull_rd(u * FIX_ONE);
  auto is_ok = [&](float x, unsigned k) { return k > 0u && k >= cut.kt && !(minp_thr > 0.f && base.prob(x) < minp_thr); };
  {
    u64 n_t = 0;
    for (int i = w0 + lane; i < w1; i += 32) { float x = vals[i]; unsigned k = key_of(x); if (k == cut.kt && is_ok(x, k)) ++n_t; }
    n_t = warp_sum_u64(n_t);
    if (lane == 0) s.warp_ties[warp] = n_t;
  }
  u64 ties_before, ties_total;
  cl_prefix_u64(c, s.warp_ties, &ties_before, &ties_total);
  for (int w = 0; w < warp; ++w) ties_before += s.warp_ties[w];
  // One element of this warp's range: is it kept, and with which weight.  `tie_run`: kept ties before
  // the row of 32; returns the weight (0 if not kept) and adds the row's ties to tie_run.
  auto weigh = [&](int i0, u64& tie_run, float* pf_out, bool* member_out) -> u64 {
    const int i = i0 + lane;
    float x = 0.f; unsigned k = 0; bool ok = false;
    if (i < w1) { x = vals[i]; k = key_of(x); ok = is_ok(x, k); }
    const bool tie = ok && k == cut.kt;
    const unsigned tm = __ballot_sync(0xffffffffu, tie);
    const u64 tie_rank = tie_run + __popc(tm & ((1u << lane) - 1));
    const bool member = ok && (k > cut.kt || tie_rank < cut.q);
    float pf = 0.f;
    if (member) { pf = pg.prob(x); if (use_sum3) pf = pf / sum3; }
    tie_run += __popc(tm);
    *pf_out = pf; *member_out = member;
    return member ? __float2ull_rd(pf * FIX_ONE) : 0ull;
  };
  // pass 1: the warp's total weight, the processed distribution if asked for, the last kept id
  int last = -1;
  {
    u64 tie_run = ties_before, lane_sum = 0;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      float pf; bool member;
      lane_sum += weigh(i0, tie_run, &pf, &member);
      if (probs && i0 + lane < w1) probs[v0 + i0 + lane] = pf;
      if (member) last = v0 + i0 + lane;
    }
    lane_sum = warp_sum_u64(lane_sum);
    if (lane == 0) s.warp_w[warp] = lane_sum;
  }
  // the weights before this CTA and in all, and (same exchange) the last kept id, for a target that
  // the rounded weights never reach
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
  if (lane == 0) s.wi[warp] = last;
  u64 w_before, w_total;
  int neg_last;
  {
    __syncthreads();
    if (threadIdx.x == 0) {
      u64 t = 0; int l = -1;
      for (int w = 0; w < SC_WARPS; ++w) { t += s.warp_w[w]; l = max(l, s.wi[w]); }
      s.xu[c.pp][0] = t; s.xi[c.pp] = l;
    }
    cg::this_cluster().sync();
    if (threadIdx.x == 0) {
      u64 b = 0, t = 0; int l = -1;
      for (int r = 0; r < SC_CL; ++r) {
        u64 x = *cg::this_cluster().map_shared_rank(&s.xu[c.pp][0], r);
        l = max(l, *cg::this_cluster().map_shared_rank(&s.xi[c.pp], r));
        if (r < c.rank) b += x;
        t += x;
      }
      s.bu[0] = b; s.bu[1] = t; s.bi = l;
    }
    __syncthreads();
    c.pp ^= 1;
    w_before = s.bu[0]; w_total = s.bu[1];
    neg_last = s.bi < 0 ? 0x7fffffff : -s.bi;
  }
  for (int w = 0; w < warp; ++w) w_before += s.warp_w[w];
  if (w_total > target) {
    // pass 2, by the one warp whose range holds the target: the first id whose running weight passes it
    if (w_before <= target && target < w_before + s.warp_w[warp]) {
      u64 tie_run = ties_before, cum = w_before;
      int tok = -1;
      for (int i0 = w0; i0 < w1 && tok < 0; i0 += 32) {
        float pf; bool member;
        u64 incl = weigh(i0, tie_run, &pf, &member);
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { u64 t = shfl_up_u64(incl, d); if (lane >= d) incl += t; }
        const unsigned over = __ballot_sync(0xffffffffu, member && cum + incl > target);
        if (over) tok = v0 + i0 + (__ffs(over) - 1);
        cum += ((u64)__shfl_sync(0xffffffffu, (unsigned)(incl >> 32), 31) << 32) | __shfl_sync(0xffffffffu, (unsigned)incl, 31);
      }
      if (lane == 0 && tok >= 0) {
        out_tokens[row] = tok;
        if (update_counts && my_counts) my_counts[tok] += 1;
      }
    }
  } else if (c.rank == 0 && threadIdx.x == 0) {
    int tok = neg_last == 0x7fffffff ? 0 : -neg_last;
    out_tokens[row] = tok;
    if (update_counts && my_counts) my_counts[tok] += 1;
  }
  cg::this_cluster().sync();                             // nobody leaves while its shared memory may be read
}

FELLM_API int fellm_sample(const float* logits, int rows, int V, const void* params, int* counts,
                           const int* bias_tok, const float* bias_val, int* out_tokens, float* out_probs,
                           int update_counts, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!logits || !params || !out_tokens || V < 1) return FELLM_ERR_ARG;
  // a cluster of eight CTAs a row where an eighth of the row fits a CTA's shared memory
  int slice = ((V + SC_CL - 1) / SC_CL + 31) / 32 * 32;
  size_t smem = (size_t)slice * sizeof(float);
  static int use_cluster = -1;
  if (use_cluster < 0) { const char* e = getenv("FELLM_B200_SAMPLE_CLUSTER"); use_cluster = (e && e[0] == '0') ? 0 : 1; }
  if (use_cluster && smem <= 160 * 1024) {
    if (smem > 32 * 1024) {
      cudaError_t ce = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ce != cudaSuccess) return (int)ce;
    }
    sample_cluster_kernel<<<dim3(rows * SC_CL), dim3(SC_THREADS), smem, stream>>>(logits, V, slice, (const RowParams*)params, counts, bias_tok,
                                                                                 bias_val, out_tokens, out_probs, update_counts);
    return launch_status();
  }
  return launch_k(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, 1, logits, V, (const RowParams*)params,
                  counts, bias_tok, bias_val, out_tokens, out_probs, update_counts);
}


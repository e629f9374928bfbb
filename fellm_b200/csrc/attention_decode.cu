// Decode attention over the paged cache, bfloat16 cache and queries, float32 softmax: one new
// token per request against thousands of cached keys.  It is bound by reading K and V once from
// HBM, so the work is split over the keys ("split-KV") until the machine is full:
//   grid = (key ranges, kv heads, rows); a CTA takes one row's one kv head and one range of keys,
//   and serves all H/G query heads of that kv head from a single read of K and V.
// Partial results (m, l, acc) of the ranges go to a scratch buffer; the CTA that finishes last for
// a (row, kv head) merges them in range order, so the result does not depend on which CTA that was.
//
// FeLLM's decode kernels keep one block per head over all keys: attention_fa2_decode_paged
// (plugins/cuda_kernels/src/oxide_kernels.rs:5107), attention_paged_batch_heads (4271).
#include "common.cuh"

#define DEC_WARPS 4
#define DEC_UNROLL 4
#define DEC_MAX_PAGES 256            // pages of one CTA's key range kept in shared memory

__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

struct DecodeArgs {
  const bf16* q; const bf16* pool; const int* block_table; const int* positions; const int* row_slot;
  bf16* out; float* scratch; int* counters;
  int max_pages, T, H, G, hd, page_tokens, layer, layers_in_group, window, split_len, max_splits;
  float scale_log2;
};

// LPK: lanes per key (a power of two >= hd/8); RR: query heads handled together (<= 4).
template <int LPK, int RR>
__global__ void __launch_bounds__(DEC_WARPS * 32) attention_decode_kernel(DecodeArgs a) {
  constexpr int KPW = 32 / LPK;                       // keys per warp pass
  __shared__ float sm_acc[DEC_WARPS][RR][LPK * 8];
  __shared__ float sm_ml[DEC_WARPS][RR][2];
  __shared__ int sm_last;
  __shared__ int sm_pages[DEC_MAX_PAGES];
  const int s = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gi = lane / LPK, li = lane % LPK, d0 = li * 8;
  const bool lane_on = d0 < a.hd;
  // positions, slots and block tables are written by copies before the step's kernels, not by a
  // kernel: they may be read before the wait
  const int pos = a.positions[t];
  const int kb = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int s_lo = kb / a.split_len, s_hi = pos / a.split_len;
  pdl_launch_dependents();
  if (s < s_lo || s > s_hi) return;
  const int n_active = s_hi - s_lo + 1;
  const int k0 = max(kb, s * a.split_len), k1 = min(pos + 1, (s + 1) * a.split_len);
  const int R = a.H / a.G;
  const int* bt = a.block_table + (size_t)a.row_slot[t] * a.max_pages;
  const int pg0 = k0 / a.page_tokens, n_pg = (k1 - 1) / a.page_tokens - pg0 + 1;
  const bool pages_in_smem = n_pg <= DEC_MAX_PAGES;
  if (pages_in_smem)
    for (int i = threadIdx.x; i < n_pg; i += DEC_WARPS * 32) sm_pages[i] = bt[pg0 + i];
  pdl_wait();
  __syncthreads();
  const size_t head_stride = (size_t)a.page_tokens * a.hd;          // one kv head's tile in a page
  const size_t v_off = (size_t)a.G * head_stride;
  const int SW = a.hd + 2;                                           // scratch record: acc[hd], m, l

  for (int r0 = 0; r0 < R; r0 += RR) {
    float qf[RR][8];
#pragma unroll
    for (int rr = 0; rr < RR; ++rr) {
      int h = g * R + r0 + rr;
      if (r0 + rr < R && lane_on) {
        uint4 v = *(const uint4*)(a.q + ((size_t)t * a.H + h) * a.hd + d0);
        unpack8(v, qf[rr]);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[rr][i] *= a.scale_log2;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[rr][i] = 0.f;
      }
    }
    float m[RR], l[RR], acc[RR][8];
#pragma unroll
    for (int rr = 0; rr < RR; ++rr) {
      m[rr] = -INFINITY; l[rr] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[rr][i] = 0.f;
    }
    // keys base + (u*WARPS + warp)*KPW + gi; the loads of the next round are in flight while this
    // round is computed
    constexpr int STEP = DEC_UNROLL * DEC_WARPS * KPW;
    auto load = [&](int base, uint4* kv, uint4* vv, bool* ok) {
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        int kj = base + (u * DEC_WARPS + warp) * KPW + gi;
        ok[u] = kj < k1;
        kv[u] = make_uint4(0, 0, 0, 0); vv[u] = kv[u];
        if (ok[u] && lane_on) {
          int lp = kj / a.page_tokens;
          int page = pages_in_smem ? sm_pages[lp - pg0] : bt[lp];
          const bf16* kp = a.pool + ((((size_t)page * a.layers_in_group + a.layer) * 2) * a.G + g) * head_stride
                           + (size_t)(kj - lp * a.page_tokens) * a.hd + d0;
          kv[u] = ldg_nc16(kp);
          vv[u] = ldg_nc16(kp + v_off);
        }
      }
    };
    auto compute = [&](const uint4* kv, const uint4* vv, const bool* ok) {
      float sc[RR][DEC_UNROLL];
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        float kf[8];
        unpack8(kv[u], kf);
#pragma unroll
        for (int rr = 0; rr < RR; ++rr) {
          float d = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) d = fmaf(qf[rr][i], kf[i], d);
#pragma unroll
          for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          sc[rr][u] = ok[u] ? d : -INFINITY;
        }
      }
#pragma unroll
      for (int rr = 0; rr < RR; ++rr) {
        float mn = m[rr];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) mn = fmaxf(mn, sc[rr][u]);
        if (mn == -INFINITY) continue;
        float corr = exp2f(m[rr] - mn);
        m[rr] = mn;
        l[rr] *= corr;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[rr][i] *= corr;
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
          float p = exp2f(sc[rr][u] - mn);
          l[rr] += p;
          float vf[8];
          unpack8(vv[u], vf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[rr][i] = fmaf(p, vf[i], acc[rr][i]);
        }
      }
    };
    {
      uint4 kA[DEC_UNROLL], vA[DEC_UNROLL], kB[DEC_UNROLL], vB[DEC_UNROLL];
      bool okA[DEC_UNROLL], okB[DEC_UNROLL];
      int base = k0;
      load(base, kA, vA, okA);
      while (true) {
        if (base + STEP < k1) load(base + STEP, kB, vB, okB);
        compute(kA, vA, okA);
        base += STEP;
        if (base >= k1) break;
        if (base + STEP < k1) load(base + STEP, kA, vA, okA);
        compute(kB, vB, okB);
        base += STEP;
        if (base >= k1) break;
      }
    }
    // merge the key groups of the warp, then the warps
#pragma unroll
    for (int rr = 0; rr < RR; ++rr) {
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) {
        float om = __shfl_xor_sync(0xffffffffu, m[rr], o), ol = __shfl_xor_sync(0xffffffffu, l[rr], o);
        float mn = fmaxf(m[rr], om);
        float c0 = mn == -INFINITY ? 0.f : exp2f(m[rr] - mn), c1 = mn == -INFINITY ? 0.f : exp2f(om - mn);
        l[rr] = l[rr] * c0 + ol * c1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float oa = __shfl_xor_sync(0xffffffffu, acc[rr][i], o);
          acc[rr][i] = acc[rr][i] * c0 + oa * c1;
        }
        m[rr] = mn;
      }
      if (gi == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_acc[warp][rr][d0 + i] = acc[rr][i];
        if (li == 0) { sm_ml[warp][rr][0] = m[rr]; sm_ml[warp][rr][1] = l[rr]; }
      }
    }
    __syncthreads();
    // CTA result per head: threads over (rr, d)
    for (int i = threadIdx.x; i < RR * a.hd; i += DEC_WARPS * 32) {
      int rr = i / a.hd, d = i - rr * a.hd;
      if (r0 + rr >= R) continue;
      float mn = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) mn = fmaxf(mn, sm_ml[w][rr][0]);
      float lt = 0.f, at = 0.f;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        float cw = sm_ml[w][rr][0] == -INFINITY ? 0.f : exp2f(sm_ml[w][rr][0] - mn);
        lt += sm_ml[w][rr][1] * cw;
        at += sm_acc[w][rr][d] * cw;
      }
      int h = g * R + r0 + rr;
      if (n_active == 1) {
        a.out[((size_t)t * a.H + h) * a.hd + d] = __float2bfloat16_rn(at / lt);
      } else {
        float* rec = a.scratch + (((size_t)t * a.H + h) * a.max_splits + (s - s_lo)) * SW;
        rec[d] = at;
        if (d == 0) { rec[a.hd] = mn; rec[a.hd + 1] = lt; }
      }
    }
    __syncthreads();
  }
  if (n_active == 1) return;

  // the last CTA of this (row, kv head) merges the ranges in order
  __threadfence();                                      // every writer publishes its records ...
  __syncthreads();                                      // ... before thread 0 counts this CTA in
  if (threadIdx.x == 0) {
    int old = atomicAdd(&a.counters[t * a.G + g], 1);
    sm_last = (old == n_active - 1);
    if (sm_last) a.counters[t * a.G + g] = 0;          // ready for the next launch
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < R * a.hd; i += DEC_WARPS * 32) {
    int r = i / a.hd, d = i - r * a.hd;
    int h = g * R + r;
    const float* rec = a.scratch + ((size_t)t * a.H + h) * a.max_splits * SW;
    float mn = -INFINITY;
    for (int j = 0; j < n_active; ++j) mn = fmaxf(mn, rec[(size_t)j * SW + a.hd]);
    float lt = 0.f, at = 0.f;
    for (int j = 0; j < n_active; ++j) {
      float cj = exp2f(rec[(size_t)j * SW + a.hd] - mn);
      lt += rec[(size_t)j * SW + a.hd + 1] * cj;
      at += rec[(size_t)j * SW + d] * cj;
    }
    a.out[((size_t)t * a.H + h) * a.hd + d] = __float2bfloat16_rn(at / lt);
  }
}

template <int LPK>
static int launch_lpk(const DecodeArgs& a, int R, cudaStream_t stream) {
  dim3 grid(a.max_splits, a.G, a.T), block(DEC_WARPS * 32, 1, 1);
  if (R == 1) return launch_k(attention_decode_kernel<LPK, 1>, grid, block, 0, stream, 1, a);
  if (R == 2) return launch_k(attention_decode_kernel<LPK, 2>, grid, block, 0, stream, 1, a);
  if (R == 3) return launch_k(attention_decode_kernel<LPK, 3>, grid, block, 0, stream, 1, a);
  return launch_k(attention_decode_kernel<LPK, 4>, grid, block, 0, stream, 1, a);
}

// scratch: float32 [T*H*max_splits*(hd+2)]; counters: int32 [T*G], zero before the first launch
// (the kernel leaves them zero).  max_splits = ceil(longest context / split_len) at least.
FELLM_API int fellm_attention_decode(const void* q, const void* pool, const int* block_table, int max_pages,
                                     const int* positions, const int* row_slot, void* out, float* scratch,
                                     int* counters, int T, int H, int G, int hd, int page_tokens, int layer,
                                     int layers_in_group, float scale, int window, int split_len,
                                     int max_splits, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd < 8 || hd > 256 || (hd % 8)) return FELLM_ERR_SIZE;
  if (G < 1 || H % G || split_len < 1 || max_splits < 1) return FELLM_ERR_SIZE;
  if (!q || !pool || !block_table || !positions || !row_slot || !out || !scratch || !counters) return FELLM_ERR_ARG;
  DecodeArgs a;
  a.q = (const bf16*)q; a.pool = (const bf16*)pool; a.block_table = block_table; a.positions = positions;
  a.row_slot = row_slot; a.out = (bf16*)out; a.scratch = scratch; a.counters = counters;
  a.max_pages = max_pages; a.T = T; a.H = H; a.G = G; a.hd = hd; a.page_tokens = page_tokens; a.layer = layer;
  a.layers_in_group = layers_in_group; a.window = window; a.split_len = split_len; a.max_splits = max_splits;
  a.scale_log2 = scale * 1.4426950408889634f;
  int R = H / G;
  int lanes = hd / 8;
  if (lanes <= 2) return launch_lpk<2>(a, R, stream);
  if (lanes <= 4) return launch_lpk<4>(a, R, stream);
  if (lanes <= 8) return launch_lpk<8>(a, R, stream);
  if (lanes <= 16) return launch_lpk<16>(a, R, stream);
  return launch_lpk<32>(a, R, stream);
}

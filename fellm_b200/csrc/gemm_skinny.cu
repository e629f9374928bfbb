// y[M,N] = x[M,K] W[N,K]^T for few rows (decode: M <= 64), bfloat16 operands, float32 sums:
// a weight-streaming kernel.
//
//  * Work item: a 16-row slab of W ("swap-AB": the slab is the A operand of mma.m16n8k16, the
//    tokens are the B operand's columns) times one slice of K.  A warp keeps two rounds of five
//    32-wide chunks (10 KB) of its item in flight.  Matrices of the decode step are small enough
//    that the launcher cuts K so finely (over the warps of a CTA, then over a thread-block
//    cluster) that every item is two rounds and the WHOLE matrix is in flight at once: one trip
//    to HBM.  Matrices too large for that (the vocabulary head) are streamed, slab after slab.
//  * A CTA stages its slice of x once, for all its warps.
//  * The first weights are requested BEFORE the kernel waits for its predecessor (programmatic
//    dependent launch): weights do not depend on the step, so HBM keeps streaming across kernel
//    boundaries.
//  * Split-K partial tiles are summed through distributed shared memory in rank order: no
//    atomics, no scratch in global memory, the same bits every run.
//  * Prologue, optional: RMSNorm of the float32 residual stream fused into the staging of x.
//  * Epilogues: store bfloat16; add into the float32 residual stream; SiLU(gate)*up over weight
//    rows interleaved in blocks of 8; float32 store (logits).
//
// FeLLM's dense product is one thread per output (plugins/cuda_kernels/src/oxide_kernels.rs:3165);
// its one fused gate/up kernel is the quantised q4k_gate_up_swiglu_multiwarp (1610); its RMSNorm
// is a kernel of its own (165).
//
// Fragment trick: the contraction does not care in which order k runs, so thread (g = lane/4,
// c = lane%4) loads 8 CONSECUTIVE k (16 bytes) of W rows g and g+8 and of token g, and feeds them
// to two MMAs as the k slots {2c,2c+1,2c+8,2c+9}; both operands use the same mapping.
#include <cooperative_groups.h>

#include "common.cuh"
namespace cg = cooperative_groups;

#define SK_ROWS 16
#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define KCHUNK 32
#define SK_U 5                       // chunks per round: 10 x 16 B per thread, two rounds in flight

enum { EPI_STORE = 0, EPI_ACC = 1, EPI_SWIGLU = 2, EPI_F32 = 3 };

__device__ __forceinline__ void mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

struct SkinnyArgs {
  const bf16* x;            // [M, K] bfloat16, or null when xf is given
  const float* xf;          // [M, K] float32 residual stream to be RMS-normed on the way in
  const float* norm_w;      // [K]
  float eps;
  const bf16* W; const float* bias; void* out;
  int M, N, K, lda, ldw, ldo, k_per_cta, xs_stride, splits, warps_k, n_tiles, tiles_per_warp;
};

template <int MT, int EPI>
__device__ __forceinline__ void epilogue_direct(const SkinnyArgs& a, float (*acc)[4], int n0, int g, int c) {
  // thread holds rows n0+g, n0+g+8 and tokens t*8 + 2c, 2c+1
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      int m = t * 8 + 2 * c + e;
      if (m >= a.M) continue;
      if (EPI == EPI_SWIGLU) {
        int n = n0 + g;                                   // gate row; the up row is n + 8
        if (n < a.N) {
          float gs = acc[t][e], us = acc[t][2 + e];
          if (a.bias) { gs += a.bias[n]; us += a.bias[n + 8]; }
          ((bf16*)a.out)[(size_t)m * a.ldo + (n0 >> 1) + g] = __float2bfloat16_rn((gs / (1.0f + expf(-gs))) * us);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          int n = n0 + g + 8 * h;
          if (n >= a.N) continue;
          float v = acc[t][2 * h + e];
          if (a.bias) v += a.bias[n];
          size_t o = (size_t)m * a.ldo + n;
          if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(v);
          else if (EPI == EPI_ACC) ((float*)a.out)[o] += v;
          else ((float*)a.out)[o] = v;
        }
      }
    }
  }
}

// MT: token tiles of 8 (M <= 8*MT).
template <int MT, int EPI>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(SkinnyArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float row_scale[MT * 8];
  constexpr int MP = MT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = a.splits > 1 ? (int)cg::this_cluster().block_rank() : 0;
  // the CTA's warps: wn = which slab of the CTA's pass, wk = which slice of the CTA's K range
  const int warps_n = SK_WARPS / a.warps_k;
  const int wn = warp / a.warps_k, wk = warp - wn * a.warps_k;
  const int k_cta = split * a.k_per_cta;
  const int k_per_warp = a.k_per_cta / a.warps_k;                    // a multiple of 32
  const int k_begin = k_cta + wk * k_per_warp;
  const int k_len = max(min(a.K, k_begin + k_per_warp) - k_begin, 0);
  const int n_chunks = (k_len + KCHUNK - 1) / KCHUNK;
  const int rounds_per_tile = max((n_chunks + SK_U - 1) / SK_U, 1);
  // this warp's slabs: first_tile, first_tile + tile_stride, ...
  const int first_tile = blockIdx.y * warps_n + wn;
  const int tile_stride = gridDim.y * warps_n;
  int my_tiles = first_tile < a.n_tiles ? (a.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const int total_rounds = my_tiles * rounds_per_tile;

  auto load_round = [&](int r, uint4* w0, uint4* w1) {
    int tl = r / rounds_per_tile, rr = r - tl * rounds_per_tile;
    int n0 = (first_tile + tl * tile_stride) * SK_ROWS;
    const bf16* p0 = a.W + (size_t)min(n0 + g, a.N - 1) * a.ldw + k_begin + c * 8;      // rows past N: clamped, never stored
    const bf16* p1 = a.W + (size_t)min(n0 + g + 8, a.N - 1) * a.ldw + k_begin + c * 8;
#pragma unroll
    for (int u = 0; u < SK_U; ++u) {
      int kk = (rr * SK_U + u) * KCHUNK;
      if (kk + c * 8 < k_len) { w0[u] = ldg_stream(p0 + kk); w1[u] = ldg_stream(p1 + kk); }
      else { w0[u] = make_uint4(0, 0, 0, 0); w1[u] = w0[u]; }
    }
  };

  // ---- weights first: they do not depend on the kernel before this one
  uint4 wA0[SK_U], wA1[SK_U], wB0[SK_U], wB1[SK_U];
  if (total_rounds > 0) load_round(0, wA0, wA1);
  if (total_rounds > 1) load_round(1, wB0, wB1);
  pdl_launch_dependents();
  pdl_wait();

  // ---- stage x[:, k_cta : k_cta + k_per_cta] as bfloat16 (rows >= M zero), normed if asked
  bf16* xs = (bf16*)smem;
  const int vec_per_row = a.k_per_cta / 8;
  if (a.xf) {
    // RMSNorm (crates/backend-cpu/src/kernels/norm.rs:6-39) over the whole row, whatever the slice
    for (int r = warp; r < a.M; r += SK_WARPS) {
      const float4* xr = (const float4*)(a.xf + (size_t)r * a.lda);
      float ss = 0.f;
      for (int i = lane; i < a.K / 4; i += 32) { float4 v = xr[i]; ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss)))); }
      ss = warp_sum(ss);
      if (lane == 0) row_scale[r] = 1.0f / sqrtf(ss / (float)a.K + a.eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < MT * 8 * vec_per_row; i += SK_THREADS) {
      int r = i / vec_per_row, v = i - r * vec_per_row;
      int k = k_cta + v * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < a.M && k < a.K) {
        const float4* xr = (const float4*)(a.xf + (size_t)r * a.lda + k);
        const float4* wr = (const float4*)(a.norm_w + k);
        float4 x0 = xr[0], x1 = xr[1], g0 = wr[0], g1 = wr[1];
        float sc = row_scale[r];
        __nv_bfloat162 p0 = __floats2bfloat162_rn((x0.x * sc) * g0.x, (x0.y * sc) * g0.y);
        __nv_bfloat162 p1 = __floats2bfloat162_rn((x0.z * sc) * g0.z, (x0.w * sc) * g0.w);
        __nv_bfloat162 p2 = __floats2bfloat162_rn((x1.x * sc) * g1.x, (x1.y * sc) * g1.y);
        __nv_bfloat162 p3 = __floats2bfloat162_rn((x1.z * sc) * g1.z, (x1.w * sc) * g1.w);
        val.x = *(unsigned*)&p0; val.y = *(unsigned*)&p1; val.z = *(unsigned*)&p2; val.w = *(unsigned*)&p3;
      }
      *(uint4*)(xs + (size_t)r * a.xs_stride + v * 8) = val;
    }
  } else {
    for (int i = threadIdx.x; i < MT * 8 * vec_per_row; i += SK_THREADS) {
      int r = i / vec_per_row, v = i - r * vec_per_row;
      int k = k_cta + v * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < a.M && k < a.K) val = *(const uint4*)(a.x + (size_t)r * a.lda + k);      // K % 8 == 0: whole vectors
      *(uint4*)(xs + (size_t)r * a.xs_stride + v * 8) = val;
    }
  }
  __syncthreads();

  // ---- rounds of SK_U chunks; the round after next is requested before this one is multiplied
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
  float* slots = (float*)(smem + (size_t)MT * 8 * a.xs_stride * sizeof(bf16));      // [warp][tile of warp][16][MP], split-K only
  const bf16* xw = xs + (size_t)g * a.xs_stride + wk * k_per_warp + c * 8;
  const bool direct = a.splits == 1 && a.warps_k == 1;

  auto compute_round = [&](int r, const uint4* w0, const uint4* w1) {
    int tl = r / rounds_per_tile, rr = r - tl * rounds_per_tile;
#pragma unroll
    for (int u = 0; u < SK_U; ++u) {
      int ch = rr * SK_U + u;
      if (ch < n_chunks) {
        unsigned fa[4] = {w0[u].x, w1[u].x, w0[u].y, w1[u].y};
        unsigned fb[4] = {w0[u].z, w1[u].z, w0[u].w, w1[u].w};
        const bf16* xr = xw + ch * KCHUNK;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          uint4 b = *(const uint4*)(xr + (size_t)t * 8 * a.xs_stride);
          mma16816(acc[t], fa, b.x, b.y);
          mma16816(acc[t], fb, b.z, b.w);
        }
      }
    }
    if (rr == rounds_per_tile - 1) {                      // the slab is done
      int n0 = (first_tile + tl * tile_stride) * SK_ROWS;
      if (direct) {
        epilogue_direct<MT, EPI>(a, acc, n0, g, c);
      } else {
        float* p = slots + ((size_t)warp * a.tiles_per_warp + tl) * SK_ROWS * MP;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          p[g * MP + t * 8 + 2 * c] = acc[t][0];
          p[g * MP + t * 8 + 2 * c + 1] = acc[t][1];
          p[(g + 8) * MP + t * 8 + 2 * c] = acc[t][2];
          p[(g + 8) * MP + t * 8 + 2 * c + 1] = acc[t][3];
        }
      }
#pragma unroll
      for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
    }
  };

  for (int r = 0; r < total_rounds; r += 2) {
    compute_round(r, wA0, wA1);
    if (r + 2 < total_rounds) load_round(r + 2, wA0, wA1);
    if (r + 1 < total_rounds) {
      compute_round(r + 1, wB0, wB1);
      if (r + 3 < total_rounds) load_round(r + 3, wB0, wB1);
    }
  }
  if (direct) return;

  // ---- split K: sum the partial slabs over the cluster's ranks and the CTA's K warps, in that
  // order; every (rank, K warp) finishes a share of each slab's rows
  if (a.splits > 1) cg::this_cluster().sync(); else __syncthreads();
  const int workers = a.splits * a.warps_k, me = split * a.warps_k + wk;
  const float* slab_slots = slots + (size_t)(wn * a.warps_k) * a.tiles_per_warp * SK_ROWS * MP;   // K warp 0 of this slab
  const size_t warp_stride = (size_t)a.tiles_per_warp * SK_ROWS * MP;
  for (int tl = 0; tl < my_tiles; ++tl) {
    int n0 = (first_tile + tl * tile_stride) * SK_ROWS;
    const float* mine = slab_slots + (size_t)tl * SK_ROWS * MP;
    const int units = (EPI == EPI_SWIGLU ? 8 : SK_ROWS) * a.M;          // outputs of the slab
    for (int i = me * 32 + lane; i < units; i += workers * 32) {
      int m, j;
      if (EPI == EPI_SWIGLU) { m = i >> 3; j = i & 7; } else { m = i >> 4; j = i & 15; }
      float v0 = 0.f, v1 = 0.f;
      for (int s = 0; s < a.splits; ++s) {
        const float* p = a.splits > 1 ? cg::this_cluster().map_shared_rank(mine, s) : mine;
        for (int w = 0; w < a.warps_k; ++w) {
          v0 += p[w * warp_stride + j * MP + m];
          if (EPI == EPI_SWIGLU) v1 += p[w * warp_stride + (j + 8) * MP + m];
        }
      }
      int n = n0 + j;
      if (n >= a.N) continue;
      if (EPI == EPI_SWIGLU) {
        if (a.bias) { v0 += a.bias[n]; v1 += a.bias[n + 8]; }
        ((bf16*)a.out)[(size_t)m * a.ldo + (n0 >> 1) + j] = __float2bfloat16_rn((v0 / (1.0f + expf(-v0))) * v1);
      } else {
        if (a.bias) v0 += a.bias[n];
        size_t o = (size_t)m * a.ldo + n;
        if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(v0);
        else if (EPI == EPI_ACC) ((float*)a.out)[o] += v0;
        else ((float*)a.out)[o] = v0;
      }
    }
  }
  if (a.splits > 1) cg::this_cluster().sync();           // nobody leaves while its slabs are being read
}

// Staged x rows are k_per_cta + pad elements apart, with the stride in bytes = 64 (mod 128): the 8
// threads of a quarter warp then read 16 bytes each from 8 different bank groups.
static inline int x_stride(int k_per_cta) { return k_per_cta + ((k_per_cta % 64 == 0) ? 32 : 0); }

static inline size_t smem_bytes(int mt, int k_per_cta, bool direct, int tiles_per_warp) {
  size_t sx = (size_t)mt * 8 * x_stride(k_per_cta) * sizeof(bf16);
  size_t sp = direct ? 0 : (size_t)SK_WARPS * tiles_per_warp * SK_ROWS * mt * 8 * sizeof(float);
  return sx + sp;
}

template <int MT, int EPI>
static int launch(const SkinnyArgs& a, int ctas_y, cudaStream_t stream) {
  size_t smem = smem_bytes(MT, a.k_per_cta, a.splits == 1 && a.warps_k == 1, a.tiles_per_warp);
  auto kern = gemm_skinny_kernel<MT, EPI>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_k_class(1, kern, dim3(a.splits, ctas_y, 1), dim3(SK_THREADS, 1, 1), smem, stream, a.splits, a);
}

template <int EPI>
static int dispatch_mt(const SkinnyArgs& a, int ctas_y, cudaStream_t s) {
  if (a.M <= 8) return launch<1, EPI>(a, ctas_y, s);
  if (a.M <= 16) return launch<2, EPI>(a, ctas_y, s);
  if (a.M <= 32) return launch<4, EPI>(a, ctas_y, s);
  return launch<8, EPI>(a, ctas_y, s);
}

// epi: 0 store bf16 [M,N]; 1 add into float32 [M,N]; 2 SiLU(gate)*up -> bf16 [M,N/2], W rows
// interleaved in blocks of 8 gate / 8 up; 3 store float32 [M,N].
// x: bfloat16 [M,K]; or x = null and xf/norm_w/eps given: float32 [M,K] normed on the way in.
FELLM_API int fellm_gemm_skinny(const void* x, const float* xf, const float* norm_w, float eps, const void* W,
                                const float* bias, void* out, int epi, int M, int N, int K, int lda, int ldw,
                                int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((!x && !xf) || !W || !out || K <= 0) return FELLM_ERR_ARG;
  if (xf && !norm_w) return FELLM_ERR_ARG;
  if (M > 64 || (K % 8) || (ldw % 8)) return FELLM_ERR_SIZE;
  if (x && (lda % 8)) return FELLM_ERR_SIZE;
  if (xf && (lda % 4)) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && (N % 16)) return FELLM_ERR_SIZE;
  int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  const size_t smem_cap = 100 * 1024;                     // two CTAs per SM
  const int resident_warps = 148 * 2 * SK_WARPS;
  const int in_flight = 2 * SK_U * KCHUNK;                // k a warp holds in flight: two rounds
  int n_tiles = ceil_div(N, SK_ROWS);
  auto round_k = [&](int k) { return ceil_div(k, KCHUNK) * KCHUNK; };
  // Plan A, "all in flight": cut K into power-of-two many slices of at most `in_flight`, first over
  // the warps of a CTA (up to 8), then over a cluster (up to 8); taken when every (slab, slice)
  // item finds a warp of its own, so that the whole matrix is requested at once.
  // Plan B, "streaming": a warp walks over whole-K slabs, two rounds ahead.
  int slices = 1;
  while (slices < 64 && ceil_div(K, slices) > in_flight) slices *= 2;
  int warps_k = slices < SK_WARPS ? slices : SK_WARPS, splits = slices / warps_k;
  bool plan_a = (long long)n_tiles * slices <= resident_warps + resident_warps / 4;
  int ctas_y = 1, tiles_per_warp = 1, k_per_cta = 0;
  if (plan_a) {
    k_per_cta = round_k(ceil_div(K, slices)) * warps_k;
    ctas_y = ceil_div(n_tiles, SK_WARPS / warps_k);
    if (ctas_y > (148 * 2) / splits) ctas_y = (148 * 2) / splits;
    tiles_per_warp = ceil_div(n_tiles, ctas_y * (SK_WARPS / warps_k));
    if (smem_bytes(mt, k_per_cta, slices == 1, tiles_per_warp) > 200 * 1024) plan_a = false;
  }
  if (!plan_a) {
    // whole K per warp where x fits; else split K over a cluster until it does (two CTAs per SM if
    // that can be had, one otherwise)
    warps_k = 1;
    bool found = false;
    for (int pass = 0; pass < 2 && !found; ++pass) {
      size_t cap = pass == 0 ? smem_cap : (size_t)200 * 1024;
      for (splits = 1; splits <= 8; splits *= 2) {
        k_per_cta = round_k(ceil_div(K, splits));
        ctas_y = ceil_div(n_tiles, SK_WARPS);
        if (ctas_y > (148 * 2) / splits) ctas_y = (148 * 2) / splits;
        if (ctas_y < 1) ctas_y = 1;
        tiles_per_warp = ceil_div(n_tiles, ctas_y * SK_WARPS);
        if (smem_bytes(mt, k_per_cta, splits == 1, tiles_per_warp) <= cap) { found = true; break; }
      }
    }
    if (!found) splits = 16;
    if (splits > 8) return FELLM_ERR_SIZE;
  }
  SkinnyArgs a;
  a.x = (const bf16*)x; a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.bias = bias; a.out = out;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldw = ldw; a.ldo = ldo; a.splits = splits;
  a.warps_k = warps_k; a.k_per_cta = k_per_cta; a.xs_stride = x_stride(k_per_cta);
  a.n_tiles = n_tiles; a.tiles_per_warp = tiles_per_warp;
  switch (epi) {
    case EPI_STORE: return dispatch_mt<EPI_STORE>(a, ctas_y, stream);
    case EPI_ACC: return dispatch_mt<EPI_ACC>(a, ctas_y, stream);
    case EPI_SWIGLU: return dispatch_mt<EPI_SWIGLU>(a, ctas_y, stream);
    case EPI_F32: return dispatch_mt<EPI_F32>(a, ctas_y, stream);
    default: return FELLM_ERR_ARG;
  }
}

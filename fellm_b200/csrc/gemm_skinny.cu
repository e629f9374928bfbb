// y[M,N] = x[M,K] W[N,K]^T for few rows (decode: M <= 64), bfloat16 operands, float32 sums:
// a weight-streaming kernel.
//
//  * A CTA owns 16 rows of W (one m16 slab, "swap-AB": W is the A operand of mma.m16n8k16, the
//    tokens are the B operand's columns).  Its 4 warps split the CTA's K range; a thread-block
//    cluster splits K further where N alone gives too few CTAs.  Partial tiles are summed through
//    shared memory in warp order and through distributed shared memory in rank order: no atomics,
//    no scratch in global memory, the same bits every run.
//  * The weights are read once from HBM with 16-byte loads straight into tensor-core fragments,
//    and the first 8 KB per warp are requested BEFORE the kernel waits for its predecessor
//    (programmatic dependent launch): weights do not depend on the step, so HBM keeps streaming
//    across kernel boundaries.
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
#define SK_WARPS 4
#define SK_THREADS (SK_WARPS * 32)
#define KCHUNK 32
#define SK_U 8                       // chunks a warp keeps in flight: 16 x 16 B per thread

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
  int M, N, K, lda, ldw, ldo, k_per_cta, xs_stride, splits;
};

// MT: token tiles of 8 (M <= 8*MT).
template <int MT, int EPI>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(SkinnyArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float row_scale[MT * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = a.splits > 1 ? (int)cg::this_cluster().block_rank() : 0;
  const int n0 = blockIdx.y * SK_ROWS;
  const int k_cta = split * a.k_per_cta;
  const int k_per_warp = a.k_per_cta / SK_WARPS;                    // a multiple of 32
  const int k_begin = k_cta + warp * k_per_warp;
  const int k_len = max(min(a.K, k_begin + k_per_warp) - k_begin, 0);
  const int n_chunks = (k_len + KCHUNK - 1) / KCHUNK;

  // ---- weights first: they do not depend on the kernel before this one
  const bf16* w0 = a.W + (size_t)min(n0 + g, a.N - 1) * a.ldw + k_begin + c * 8;     // rows past N: clamped, never stored
  const bf16* w1 = a.W + (size_t)min(n0 + g + 8, a.N - 1) * a.ldw + k_begin + c * 8;
  uint4 a0[SK_U], a1[SK_U];
#pragma unroll
  for (int u = 0; u < SK_U; ++u) {
    if (u * KCHUNK + c * 8 < k_len) { a0[u] = ldg_stream(w0 + u * KCHUNK); a1[u] = ldg_stream(w1 + u * KCHUNK); }
    else { a0[u] = make_uint4(0, 0, 0, 0); a1[u] = a0[u]; }
  }
  pdl_launch_dependents();
  pdl_wait();

  // ---- stage x[:, k_cta : k_cta + k_per_cta] as bfloat16 (rows >= M zero), normed if asked
  bf16* xs = (bf16*)smem;
  const int vec_per_row = a.k_per_cta / 8;
  if (a.xf) {
    // RMSNorm (crates/backend-cpu/src/kernels/norm.rs:6-39): the CTA holds the whole K range
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

  // ---- this warp's K slice of the CTA's 16 rows
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
  const bf16* xw = xs + (size_t)g * a.xs_stride + warp * k_per_warp + c * 8;
  for (int ch0 = 0; ch0 < n_chunks; ch0 += SK_U) {
    if (ch0 > 0) {
#pragma unroll
      for (int u = 0; u < SK_U; ++u) {
        if ((ch0 + u) * KCHUNK + c * 8 < k_len) { a0[u] = ldg_stream(w0 + (ch0 + u) * KCHUNK); a1[u] = ldg_stream(w1 + (ch0 + u) * KCHUNK); }
        else { a0[u] = make_uint4(0, 0, 0, 0); a1[u] = a0[u]; }
      }
    }
#pragma unroll
    for (int u = 0; u < SK_U; ++u) {
      if (ch0 + u < n_chunks) {
        unsigned fa[4] = {a0[u].x, a1[u].x, a0[u].y, a1[u].y};
        unsigned fb[4] = {a0[u].z, a1[u].z, a0[u].w, a1[u].w};
        const bf16* xr = xw + (ch0 + u) * KCHUNK;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          uint4 b = *(const uint4*)(xr + (size_t)t * 8 * a.xs_stride);
          mma16816(acc[t], fa, b.x, b.y);
          mma16816(acc[t], fb, b.z, b.w);
        }
      }
    }
  }

  // ---- warps' partial tiles -> shared memory -> the CTA's tile red[row][token]
  __syncthreads();                                   // x staging is done with; reuse the buffer
  constexpr int MP = MT * 8;
  float* part = (float*)smem;                        // [warp][16][MP]
  float* red = part + SK_WARPS * SK_ROWS * MP;       // [16][MP]
  {
    float* p = part + (size_t)warp * SK_ROWS * MP;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      p[g * MP + t * 8 + 2 * c] = acc[t][0];
      p[g * MP + t * 8 + 2 * c + 1] = acc[t][1];
      p[(g + 8) * MP + t * 8 + 2 * c] = acc[t][2];
      p[(g + 8) * MP + t * 8 + 2 * c + 1] = acc[t][3];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < SK_ROWS * MP; i += SK_THREADS) {
    float v = part[i];
#pragma unroll
    for (int w = 1; w < SK_WARPS; ++w) v += part[w * SK_ROWS * MP + i];
    red[i] = v;
  }
  if (a.splits > 1) cg::this_cluster().sync(); else __syncthreads();

  // ---- sum over the cluster in rank order, epilogue; each rank finishes a share of the rows
  if (EPI == EPI_SWIGLU) {
    // rows 0-7 are gate, rows 8-15 the up rows of the same 8 features
    const int per_rank = 8 / a.splits, j0 = split * per_rank;
    for (int i = threadIdx.x; i < per_rank * a.M; i += SK_THREADS) {
      int m = i / per_rank, j = j0 + (i - m * per_rank);
      float gs = 0.f, us = 0.f;
      for (int s = 0; s < a.splits; ++s) {
        const float* p = a.splits > 1 ? cg::this_cluster().map_shared_rank(red, s) : red;
        gs += p[j * MP + m];
        us += p[(j + 8) * MP + m];
      }
      int n = n0 + j;
      if (n < a.N) {
        if (a.bias) { gs += a.bias[n]; us += a.bias[n + 8]; }
        ((bf16*)a.out)[(size_t)m * a.ldo + (n0 >> 1) + j] = __float2bfloat16_rn((gs / (1.0f + expf(-gs))) * us);
      }
    }
  } else {
    const int per_rank = SK_ROWS / a.splits, j0 = split * per_rank;
    for (int i = threadIdx.x; i < per_rank * a.M; i += SK_THREADS) {
      int m = i / per_rank, j = j0 + (i - m * per_rank);
      float v = 0.f;
      for (int s = 0; s < a.splits; ++s) {
        const float* p = a.splits > 1 ? cg::this_cluster().map_shared_rank(red, s) : red;
        v += p[j * MP + m];
      }
      int n = n0 + j;
      if (n < a.N) {
        if (a.bias) v += a.bias[n];
        size_t o = (size_t)m * a.ldo + n;
        if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(v);
        else if (EPI == EPI_ACC) ((float*)a.out)[o] += v;
        else ((float*)a.out)[o] = v;
      }
    }
  }
  if (a.splits > 1) cg::this_cluster().sync();         // nobody leaves while its tile is being read
}

// Staged x rows are k_per_cta + pad elements apart, with the stride in bytes = 64 (mod 128): the 8
// threads of a quarter warp then read 16 bytes each from 8 different bank groups.
static inline int x_stride(int k_per_cta) { return k_per_cta + ((k_per_cta % 64 == 0) ? 32 : 0); }

static inline size_t smem_bytes(int mt, int k_per_cta) {
  size_t sx = (size_t)mt * 8 * x_stride(k_per_cta) * sizeof(bf16);
  size_t sp = (size_t)(SK_WARPS + 1) * SK_ROWS * mt * 8 * sizeof(float);
  return sx > sp ? sx : sp;
}

template <int MT, int EPI>
static int launch(const SkinnyArgs& a, cudaStream_t stream) {
  size_t smem = smem_bytes(MT, a.k_per_cta);
  auto kern = gemm_skinny_kernel<MT, EPI>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_k(kern, dim3(a.splits, ceil_div(a.N, SK_ROWS), 1), dim3(SK_THREADS, 1, 1), smem, stream, a.splits, a);
}

template <int EPI>
static int dispatch_mt(const SkinnyArgs& a, cudaStream_t s) {
  if (a.M <= 8) return launch<1, EPI>(a, s);
  if (a.M <= 16) return launch<2, EPI>(a, s);
  if (a.M <= 32) return launch<4, EPI>(a, s);
  return launch<8, EPI>(a, s);
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
  if (xf && ((lda % 4) || (K % 8))) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && (N % 16)) return FELLM_ERR_SIZE;
  int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  const size_t smem_cap = 160 * 1024;
  // split K over a cluster while N alone gives too few CTAs and the slices stay worth a warp's while
  int tiles = ceil_div(N, SK_ROWS);
  int splits = 1;
  auto kpc = [&](int s) { return ceil_div(ceil_div(K, s), SK_WARPS * KCHUNK) * SK_WARPS * KCHUNK; };
  if (!xf) {
    while (splits < 8 && tiles * splits < 256 && K / (splits * 2) >= 256) splits *= 2;
  }
  while (splits < 8 && smem_bytes(mt, kpc(splits)) > smem_cap && !xf) splits *= 2;
  if (smem_bytes(mt, kpc(splits)) > 200 * 1024) return FELLM_ERR_SIZE;
  SkinnyArgs a;
  a.x = (const bf16*)x; a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.bias = bias; a.out = out;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldw = ldw; a.ldo = ldo; a.splits = splits;
  a.k_per_cta = kpc(splits); a.xs_stride = x_stride(a.k_per_cta);
  switch (epi) {
    case EPI_STORE: return dispatch_mt<EPI_STORE>(a, stream);
    case EPI_ACC: return dispatch_mt<EPI_ACC>(a, stream);
    case EPI_SWIGLU: return dispatch_mt<EPI_SWIGLU>(a, stream);
    case EPI_F32: return dispatch_mt<EPI_F32>(a, stream);
    default: return FELLM_ERR_ARG;
  }
}

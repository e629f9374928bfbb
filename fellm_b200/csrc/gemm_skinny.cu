// y[M,N] = x[M,K] W[N,K]^T for few rows (decode: M <= 64), bfloat16 operands, float32 sums:
// a weight-streaming kernel.  The weights are read once from HBM with 16-byte loads straight into
// tensor-core fragments ("swap-AB": a 16-row slab of W is the A operand of mma.m16n8k16, the
// tokens are the B operand's 8 columns), K is split over a thread-block cluster whose partial
// tiles are summed through distributed shared memory in rank order (no atomics, no scratch in
// global memory, the same bits every run), and the epilogue is fused: store, add into the float32
// residual stream, or SiLU(gate)*up.
//
// FeLLM's dense product is one thread per output (plugins/cuda_kernels/src/oxide_kernels.rs:3165);
// its one fused gate/up kernel is the quantised q4k_gate_up_swiglu_multiwarp (1610).
//
// Fragment trick: the contraction does not care in which order k runs, so thread (g = lane/4,
// c = lane%4) loads 8 CONSECUTIVE k (16 bytes) of W rows g and g+8 and of token g, and feeds them
// to two MMAs as the k slots {2c,2c+1,2c+8,2c+9}; both operands use the same mapping.
#include <cooperative_groups.h>

#include "common.cuh"
namespace cg = cooperative_groups;

#define ROWS_PER_WARP 16
#define WARPS 4
#define ROWS_PER_CTA (ROWS_PER_WARP * WARPS)
#define KCHUNK 32

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

// MT: token tiles of 8 (M <= 8*MT).
template <int MT, int EPI>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, const float* __restrict__ bias,
                   void* __restrict__ out, int M, int N, int K, int lda, int ldw, int ldo, int k_per_cta,
                   int xs_stride, int splits) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = splits > 1 ? (int)cg::this_cluster().block_rank() : 0;
  const int n_tile0 = blockIdx.y * ROWS_PER_CTA;
  const int k_begin = split * k_per_cta;
  const int k_end = min(K, k_begin + k_per_cta);
  const int k_len = max(k_end - k_begin, 0);

  // ---- stage x[:, k_begin:k_end] as bf16, rows >= M zero
  bf16* xs = (bf16*)smem;
  {
    const int vec_per_row = k_per_cta / 8;
    for (int i = threadIdx.x; i < MT * 8 * vec_per_row; i += WARPS * 32) {
      int r = i / vec_per_row, v = i - r * vec_per_row;
      uint4 val = make_uint4(0, 0, 0, 0);
      int k = k_begin + v * 8;
      if (r < M && k < k_end) val = *(const uint4*)(x + (size_t)r * lda + k);      // K % 8 == 0: whole vectors
      *(uint4*)(xs + (size_t)r * xs_stride + v * 8) = val;
    }
  }
  __syncthreads();

  // ---- stream this warp's 16 rows of W over the CTA's K range
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
  const int row0 = n_tile0 + warp * ROWS_PER_WARP + g;
  const int row1 = row0 + 8;
  const bf16* w0 = W + (size_t)min(row0, N - 1) * ldw + k_begin + c * 8;       // rows past N are clamped, never stored
  const bf16* w1 = W + (size_t)min(row1, N - 1) * ldw + k_begin + c * 8;
  const int n_chunks = (k_len + KCHUNK - 1) / KCHUNK;
  constexpr int U = 8;
  for (int ch0 = 0; ch0 < n_chunks; ch0 += U) {
    uint4 a0[U], a1[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int kk = (ch0 + u) * KCHUNK + c * 8;
      if (kk < k_len) { a0[u] = ldg_stream(w0 + (ch0 + u) * KCHUNK); a1[u] = ldg_stream(w1 + (ch0 + u) * KCHUNK); }
      else { a0[u] = make_uint4(0, 0, 0, 0); a1[u] = a0[u]; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ch0 + u < n_chunks) {
        unsigned fa[4] = {a0[u].x, a1[u].x, a0[u].y, a1[u].y};
        unsigned fb[4] = {a0[u].z, a1[u].z, a0[u].w, a1[u].w};
        const bf16* xr = xs + (size_t)g * xs_stride + (ch0 + u) * KCHUNK + c * 8;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          uint4 b = *(const uint4*)(xr + (size_t)t * 8 * xs_stride);
          mma16816(acc[t], fa, b.x, b.y);
          mma16816(acc[t], fb, b.z, b.w);
        }
      }
    }
  }

  // ---- partial tile to shared memory: part[row in CTA][token]
  __syncthreads();                                   // x staging is done with; reuse the buffer
  float* part = (float*)smem;
  constexpr int MP = MT * 8;
  {
    int r = warp * ROWS_PER_WARP + g;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      part[(size_t)r * MP + t * 8 + 2 * c] = acc[t][0];
      part[(size_t)r * MP + t * 8 + 2 * c + 1] = acc[t][1];
      part[(size_t)(r + 8) * MP + t * 8 + 2 * c] = acc[t][2];
      part[(size_t)(r + 8) * MP + t * 8 + 2 * c + 1] = acc[t][3];
    }
  }
  if (splits > 1) cg::this_cluster().sync(); else __syncthreads();

  // ---- reduce over the cluster in rank order and apply the epilogue; rank s owns a slice of rows
  const int rows_per_rank = ROWS_PER_CTA / splits;
  const int r_begin = split * rows_per_rank;
  if (EPI == EPI_SWIGLU) {
    // rows come in blocks of 16: 8 gate rows then the 8 up rows of the same features
    const int feats = rows_per_rank / 2;               // rows_per_rank is a multiple of 16
    for (int i = threadIdx.x; i < feats * M; i += WARPS * 32) {
      int m = i / feats, j = i - m * feats;
      int blk = j >> 3, within = j & 7;
      int rg = r_begin + blk * 16 + within, ru = rg + 8;
      float gsum = 0.f, usum = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float* p = splits > 1 ? cg::this_cluster().map_shared_rank(part, s) : part;
        gsum += p[(size_t)rg * MP + m];
        usum += p[(size_t)ru * MP + m];
      }
      int n_gate = n_tile0 + rg;                         // row of the interleaved weight
      if (n_gate < N) {
        int f = (n_gate >> 4) * 8 + (n_gate & 7);
        if (bias) { gsum += bias[n_gate]; usum += bias[n_gate + 8]; }
        ((bf16*)out)[(size_t)m * ldo + f] = __float2bfloat16_rn((gsum / (1.0f + expf(-gsum))) * usum);
      }
    }
  } else {
    for (int i = threadIdx.x; i < rows_per_rank * M; i += WARPS * 32) {
      int m = i / rows_per_rank, j = i - m * rows_per_rank;
      int r = r_begin + j, n = n_tile0 + r;
      float v = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float* p = splits > 1 ? cg::this_cluster().map_shared_rank(part, s) : part;
        v += p[(size_t)r * MP + m];
      }
      if (n < N) {
        if (bias) v += bias[n];
        size_t o = (size_t)m * ldo + n;
        if (EPI == EPI_STORE) ((bf16*)out)[o] = __float2bfloat16_rn(v);
        else if (EPI == EPI_ACC) ((float*)out)[o] += v;
        else ((float*)out)[o] = v;
      }
    }
  }
  if (splits > 1) cg::this_cluster().sync();           // nobody leaves while its tile is being read
}

// Staged x rows are k_per_cta + pad elements apart, with the stride in bytes = 64 (mod 128): the 8
// threads of a quarter warp then read 16 bytes each from 8 different bank groups.
static inline int x_stride(int k_per_cta) { return k_per_cta + ((k_per_cta % 64 == 0) ? 32 : 0); }

template <int MT, int EPI>
static int launch(const bf16* x, const bf16* W, const float* bias, void* out, int M, int N, int K, int lda,
                  int ldw, int ldo, int splits, int k_per_cta, cudaStream_t stream) {
  int xs_stride = x_stride(k_per_cta);
  size_t smem_x = (size_t)MT * 8 * xs_stride * sizeof(bf16);
  size_t smem_p = (size_t)ROWS_PER_CTA * MT * 8 * sizeof(float);
  size_t smem = smem_x > smem_p ? smem_x : smem_p;
  auto kern = gemm_skinny_kernel<MT, EPI>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, ceil_div(N, ROWS_PER_CTA), 1);
  cfg.blockDim = dim3(WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = splits > 1 ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, x, W, bias, out, M, N, K, lda, ldw, ldo, k_per_cta, xs_stride, splits);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}

template <int EPI>
static int dispatch_mt(const bf16* x, const bf16* W, const float* bias, void* out, int M, int N, int K, int lda,
                       int ldw, int ldo, int splits, int k_per_cta, cudaStream_t s) {
  if (M <= 8) return launch<1, EPI>(x, W, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, s);
  if (M <= 16) return launch<2, EPI>(x, W, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, s);
  if (M <= 32) return launch<4, EPI>(x, W, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, s);
  return launch<8, EPI>(x, W, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, s);
}

// epi: 0 store bf16 [M,N]; 1 add into float32 [M,N]; 2 SiLU(gate)*up -> bf16 [M,N/2], W rows
// interleaved in blocks of 8 gate / 8 up; 3 store float32 [M,N].
FELLM_API int fellm_gemm_skinny(const void* x, const void* W, const float* bias, void* out, int epi, int M,
                                int N, int K, int lda, int ldw, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!x || !W || !out || K <= 0) return FELLM_ERR_ARG;
  if (M > 64 || (K % 8) || (lda % 8) || (ldw % 8)) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && (N % 16)) return FELLM_ERR_SIZE;
  // split K over a cluster until the machine is covered; each CTA's slice is a multiple of 32
  int tiles = ceil_div(N, ROWS_PER_CTA);
  int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  int splits = 1, max_splits = epi == EPI_SWIGLU ? 4 : 8;      // a rank reduces whole gate/up blocks of 16 rows
  while (splits < max_splits && tiles * splits < 148 * 2 && K / (splits * 2) >= 64) splits *= 2;
  int k_per_cta = ceil_div(ceil_div(K, splits), KCHUNK) * KCHUNK;
  // the staged x slice must fit shared memory
  while ((size_t)mt * 8 * x_stride(k_per_cta) * 2 > 160 * 1024 && splits < max_splits) {
    splits *= 2;
    k_per_cta = ceil_div(ceil_div(K, splits), KCHUNK) * KCHUNK;
  }
  if ((size_t)mt * 8 * x_stride(k_per_cta) * 2 > 200 * 1024) return FELLM_ERR_SIZE;
  const bf16* xb = (const bf16*)x; const bf16* wb = (const bf16*)W;
  switch (epi) {
    case EPI_STORE: return dispatch_mt<EPI_STORE>(xb, wb, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, stream);
    case EPI_ACC: return dispatch_mt<EPI_ACC>(xb, wb, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, stream);
    case EPI_SWIGLU: return dispatch_mt<EPI_SWIGLU>(xb, wb, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, stream);
    case EPI_F32: return dispatch_mt<EPI_F32>(xb, wb, bias, out, M, N, K, lda, ldw, ldo, splits, k_per_cta, stream);
    default: return FELLM_ERR_ARG;
  }
}

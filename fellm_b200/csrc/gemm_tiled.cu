// C[M,N] = A[M,K] W[N,K]^T for many rows, bfloat16 operands, float32 sums, on the warp-level
// tensor-core path (mma.sync.m16n8k16, ldmatrix, cp.async): the product for shapes the tcgen05
// kernel does not take, and its yardstick.  128x128x32 tiles, 8 warps of 64x32, three stages.
// Epilogues as in gemm_skinny.cu: store, add into the float32 residual stream, SiLU(gate)*up over
// weight rows interleaved in blocks of 8, float32 store.
//
// FeLLM counterpart: bf16_matmul_rows (plugins/cuda_kernels/src/oxide_kernels.rs:3165).
#include "common.cuh"

#define TBM 128
#define TBN 128
#define TBK 32
#define TSTAGES 3
#define TTHREADS 256

enum { EPI_STORE = 0, EPI_ACC = 1, EPI_SWIGLU = 2, EPI_F32 = 3 };

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = pred ? 16 : 0;                      // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A tile row holds 32 bf16 = four 16-byte chunks; chunk c of row r lives at chunk c ^ ((r>>1)&3),
// which spreads the 8 rows an ldmatrix reads over all banks.
__device__ __forceinline__ int swz(int row, int chunk) { return row * 4 + (chunk ^ ((row >> 1) & 3)); }

template <int EPI>
__global__ void __launch_bounds__(TTHREADS)
gemm_tiled_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, const float* __restrict__ bias,
                  void* __restrict__ out, int M, int N, int K, int lda, int ldw, int ldo) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_TILED);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* sA = (uint4*)smem_raw;                            // [stage][128 rows * 4 chunks]
  uint4* sB = sA + TSTAGES * TBM * 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wn = warp & 3;                 // 2 x 4 warps: 64 rows x 32 cols each
  const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;
  const int k_tiles = (K + TBK - 1) / TBK;

  auto load_stage = [&](int stage, int kt) {
    // 512 chunks per operand, 2 per thread each
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int ch = tid + i * TTHREADS;
      int row = ch >> 2, c = ch & 3;
      int k = kt * TBK + c * 8;
      bool kin = k < K;
      int gm = m0 + row, gn = n0 + row;
      cp_async16(&sA[stage * TBM * 4 + swz(row, c)], A + (size_t)min(gm, M - 1) * lda + (kin ? k : 0), kin && gm < M);
      cp_async16(&sB[stage * TBN * 4 + swz(row, c)], W + (size_t)min(gn, N - 1) * ldw + (kin ? k : 0), kin && gn < N);
    }
  };

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

#pragma unroll
  for (int s = 0; s < TSTAGES - 1; ++s) {
    if (s < k_tiles) load_stage(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    cp_async_wait<TSTAGES - 2>();
    __syncthreads();
    if (kt + TSTAGES - 1 < k_tiles) load_stage((kt + TSTAGES - 1) % TSTAGES, kt + TSTAGES - 1);
    cp_async_commit();
    const uint4* a_st = sA + (kt % TSTAGES) * TBM * 4;
    const uint4* b_st = sB + (kt % TSTAGES) * TBN * 4;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {                       // two k16 steps per tile
      unsigned af[4][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // matrices: (rows 0-7,k lo) (rows 8-15,k lo) (rows 0-7,k hi) (rows 8-15,k hi)
        int row = wm * 64 + i * 16 + (lane & 15);
        int chunk = ks * 2 + (lane >> 4);
        ldmatrix_x4(af[i], &a_st[swz(row, chunk)]);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        // two n8 tiles: (n 0-7,k lo) (n 0-7,k hi) (n 8-15,k lo) (n 8-15,k hi)
        int row = wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3);
        int chunk = ks * 2 + ((lane >> 3) & 1);
        unsigned r[4];
        ldmatrix_x4(r, &b_st[swz(row, chunk)]);
        bfr[2 * j][0] = r[0]; bfr[2 * j][1] = r[1]; bfr[2 * j + 1][0] = r[2]; bfr[2 * j + 1][1] = r[3];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma16816(acc[i][j], af[i], bfr[j][0], bfr[j][1]);
    }
  }
  cp_async_wait<0>();

  // ---- epilogue: thread holds rows g, g+8 and columns 2c, 2c+1 of every 16x8 tile
  const int g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      int m = m0 + wm * 64 + i * 16 + g + half * 8;
      if (m >= M) continue;
      if (EPI == EPI_SWIGLU) {
        // columns come in blocks of 16: 8 gate then the 8 up of the same features = n8 tiles 2j, 2j+1
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
          int n = n0 + wn * 32 + j * 8 + 2 * c;            // gate column
          if (n < N) {
            int f = (n >> 4) * 8 + (n & 7);
            float g0 = acc[i][j][half * 2], g1 = acc[i][j][half * 2 + 1];
            float u0 = acc[i][j + 1][half * 2], u1 = acc[i][j + 1][half * 2 + 1];
            if (bias) { g0 += bias[n]; g1 += bias[n + 1]; u0 += bias[n + 8]; u1 += bias[n + 9]; }
            __nv_bfloat162 v = __floats2bfloat162_rn((g0 / (1.0f + expf(-g0))) * u0, (g1 / (1.0f + expf(-g1))) * u1);
            *(__nv_bfloat162*)((bf16*)out + (size_t)m * ldo + f) = v;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int n = n0 + wn * 32 + j * 8 + 2 * c;
          float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (n + e >= N) continue;
            float v = e ? v1 : v0;
            if (bias) v += bias[n + e];
            size_t o = (size_t)m * ldo + n + e;
            if (EPI == EPI_STORE) ((bf16*)out)[o] = __float2bfloat16_rn(v);
            else if (EPI == EPI_ACC) ((float*)out)[o] += v;
            else ((float*)out)[o] = v;
          }
        }
      }
    }
  }
}

template <int EPI>
static int launch(const bf16* A, const bf16* W, const float* bias, void* out, int M, int N, int K, int lda,
                  int ldw, int ldo, cudaStream_t stream) {
  size_t smem = (size_t)TSTAGES * (TBM + TBN) * 4 * sizeof(uint4);
  auto kern = gemm_tiled_kernel<EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(ceil_div(N, TBN), ceil_div(M, TBM));
  kern<<<grid, TTHREADS, smem, stream>>>(A, W, bias, out, M, N, K, lda, ldw, ldo);
  return launch_status();
}

FELLM_API int fellm_gemm_tiled(const void* A, const void* W, const float* bias, void* out, int epi, int M, int N,
                               int K, int lda, int ldw, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!A || !W || !out || K <= 0) return FELLM_ERR_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8)) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && ((N % 16) || (ldo % 2))) return FELLM_ERR_SIZE;
  const bf16* a = (const bf16*)A; const bf16* w = (const bf16*)W;
  switch (epi) {
    case EPI_STORE: return launch<EPI_STORE>(a, w, bias, out, M, N, K, lda, ldw, ldo, stream);
    case EPI_ACC: return launch<EPI_ACC>(a, w, bias, out, M, N, K, lda, ldw, ldo, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU>(a, w, bias, out, M, N, K, lda, ldw, ldo, stream);
    case EPI_F32: return launch<EPI_F32>(a, w, bias, out, M, N, K, lda, ldw, ldo, stream);
    default: return FELLM_ERR_ARG;
  }
}

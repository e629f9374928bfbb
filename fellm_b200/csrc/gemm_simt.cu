// C[M,N] = A[M,K] * W[N,K]^T on CUDA cores with float32 FMA: the true 32-bit matrix product
// (no TF32, no reduced-precision staging), and the product for any mix of bfloat16/float32
// operands that the tensor-core kernels do not take.
//
// FeLLM counterpart: bf16_matmul_rows / f32_matmul_rows, one thread per output
// (plugins/cuda_kernels/src/oxide_kernels.rs:3165-3225).  Like them, every output element is one
// chain acc = fma(a[m,k], w[n,k], acc) for k = 0..K-1, so its value does not depend on M, on the
// tile it falls in, or on what else is in the batch.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

// EPI 0: C = acc (+bias);  EPI 1: C(float) = C + acc (+bias)   (residual accumulate)
template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_tn_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                    TO* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_SIMT);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  int tid = threadIdx.x;
  int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread; k fastest for coalescing
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = tid + i * 256;
      int r = e >> 4, kk = e & 15;
      int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? to_f(A[(size_t)gm * lda + gk]) : 0.f;
      Ws[kk][r] = (gn < N && gk < K) ? to_f(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      size_t o = (size_t)gm * ldc + gn;
      if (EPI == 1) C[o] = from_f<TO>(to_f(C[o]) + v);
      else C[o] = from_f<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
static int launch_epi(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                      int lda, int ldw, int ldc, int accumulate, cudaStream_t s) {
  dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
  if (accumulate)
    gemm_tn_simt_kernel<TA, TW, TO, 1><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, bias, (TO*)C, M, N, K, lda, ldw, ldc);
  else
    gemm_tn_simt_kernel<TA, TW, TO, 0><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, bias, (TO*)C, M, N, K, lda, ldw, ldc);
  return launch_status();
}

// dtype codes: 0 = float32, 1 = bfloat16.  accumulate needs a float32 C.
FELLM_API int fellm_gemm_simt(const void* A, int a_dt, const void* W, int w_dt, const float* bias,
                              void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                              int accumulate, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (!A || !W || !C || K <= 0) return FELLM_ERR_ARG;
  if (accumulate && c_dt != 0) return FELLM_ERR_ARG;
  int key = a_dt * 4 + w_dt * 2 + c_dt;
  switch (key) {
    case 0: return launch_epi<float, float, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, s);
    case 2: return launch_epi<float, bf16, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, s);
    case 4: return launch_epi<bf16, float, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, s);
    case 5: return launch_epi<bf16, float, bf16>(A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, s);
    case 6: return launch_epi<bf16, bf16, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, s);
    case 7: return launch_epi<bf16, bf16, bf16>(A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, s);
    default: return FELLM_ERR_ARG;   // float32 activations never round down to a bfloat16 result
  }
}

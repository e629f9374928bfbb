// Embedding gather, RMSNorm, SiLU-gate, row gather.
//
// FeLLM counterparts (plugins/cuda_kernels/src/oxide_kernels.rs): embedding_bf16_rows (3140),
// rmsnorm_group (165), silu_gate (67).  The residual stream is float32 in both engine dtypes;
// norms read it and write the engine's activation dtype.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                  float* __restrict__ out, int d, int vocab, int* __restrict__ status) {
  FELLM_TRACE_SCOPE(TRACE_EMBED_ROWS);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();                 // the residual buffer may still be read by the step before
  int row = blockIdx.x;
  int tok = tokens[row];
  float* o = out + (size_t)row * d;
  if (tok < 0 || tok >= vocab) {          // never read outside the table: record and write zeros
    if (threadIdx.x == 0 && status) atomicExch(status, 1);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* src = table + (size_t)tok * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f(src[i]);
}

FELLM_API int fellm_embed_rows(const int* tokens, const void* table, int table_is_bf16, float* out,
                               int rows, int d, int vocab, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!tokens || !table || !out) return FELLM_ERR_ARG;
  int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
  if (table_is_bf16)
    return launch_k_class(launch_class_for_rows(rows, 2), embed_rows_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, 1, tokens, (const bf16*)table, out, d, vocab, status);
  return launch_k_class(launch_class_for_rows(rows, 2), embed_rows_kernel<float>, dim3(rows), dim3(threads), 0, stream, 1, tokens, (const float*)table, out, d, vocab, status);
}

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w, product order (x*scale)*w, all in float32.
// One block per output row; the reduction order depends on d and the block size only, so a row's
// result does not depend on which other rows are in the batch.
template <typename TO, int THREADS>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TO* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
  FELLM_TRACE_SCOPE(TRACE_RMSNORM);
  __shared__ float partial[THREADS / 32];
  __shared__ float scale_s;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  int orow = blockIdx.x;
  int irow = rows ? rows[orow] : orow;
  const float* xr = x + (size_t)irow * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) { float v = xr[i]; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) t += partial[i];
    scale_s = 1.0f / sqrtf(t / (float)d + eps);
  }
  __syncthreads();
  float scale = scale_s;
  TO* o = out + (size_t)orow * d;
  for (int i = threadIdx.x; i < d; i += THREADS) o[i] = from_f<TO>((xr[i] * scale) * w[i]);
}

__device__ __forceinline__ void store4(float* o, float a, float b, float c, float e) { *(float4*)o = make_float4(a, b, c, e); }
__device__ __forceinline__ void store4(bf16* o, float a, float b, float c, float e) {
  __nv_bfloat162 p0 = __floats2bfloat162_rn(a, b), p1 = __floats2bfloat162_rn(c, e);
  uint2 v; v.x = *(unsigned*)&p0; v.y = *(unsigned*)&p1;
  *(uint2*)o = v;
}

// d % 4 == 0: a warp per row, 16-byte loads; up to VPL vectors of a lane stay in registers between
// the sum and the scaling (rows longer than 128*VPL are read a second time).  A row's sum has the
// same order whatever else is in the batch.
template <typename TO, int VPL>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows, int n_rows, int d, float eps) {
  FELLM_TRACE_SCOPE(TRACE_RMSNORM_VEC);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  const int lane = threadIdx.x & 31;
  const int orow = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (orow >= n_rows) return;
  const int irow = rows ? rows[orow] : orow;
  const float4* xr = (const float4*)(x + (size_t)irow * d);
  const float4* wr = (const float4*)w;
  const int nv = d >> 2;
  float4 keep[VPL];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int i = lane + j * 32;
    keep[j] = i < nv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j)
    ss = fmaf(keep[j].x, keep[j].x, fmaf(keep[j].y, keep[j].y, fmaf(keep[j].z, keep[j].z, fmaf(keep[j].w, keep[j].w, ss))));
  for (int i = lane + VPL * 32; i < nv; i += 32) {
    float4 v = xr[i];
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)d + eps);
  TO* o = out + (size_t)orow * d;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int i = lane + j * 32;
    if (i < nv) {
      float4 g = wr[i];
      store4(o + 4 * i, (keep[j].x * scale) * g.x, (keep[j].y * scale) * g.y, (keep[j].z * scale) * g.z, (keep[j].w * scale) * g.w);
    }
  }
  for (int i = lane + VPL * 32; i < nv; i += 32) {
    float4 v = xr[i], g = wr[i];
    store4(o + 4 * i, (v.x * scale) * g.x, (v.y * scale) * g.y, (v.z * scale) * g.z, (v.w * scale) * g.w);
  }
}

// RMSNorm as a kernel of its own runs where the products do not take it in (17 rows and more): launched as a
// programmatic dependent from FELLM_B200_NORM_PDL_ROWS rows on, its launch hides under the product in front.
static int norm_class(int rows) {
  static int from = -1;
  if (from < 0) { const char* e = getenv("FELLM_B200_NORM_PDL_ROWS"); from = e ? atoi(e) : 17; }
  return rows >= from ? 1 : 0;
}

FELLM_API int fellm_rmsnorm(const float* x, const float* w, void* out, int out_is_bf16,
                            const int* rows, int n_out_rows, int d, float eps, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (!x || !w || !out) return FELLM_ERR_ARG;
  if (d % 4 == 0 && d >= 128) {
    const int warps = 4;
    dim3 vgrid((n_out_rows + warps - 1) / warps);
    if (d <= 1024) {
      if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<bf16, 8>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (bf16*)out, rows, n_out_rows, d, eps);
      return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<float, 8>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (float*)out, rows, n_out_rows, d, eps);
    }
    if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<bf16, 16>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (bf16*)out, rows, n_out_rows, d, eps);
    return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<float, 16>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (float*)out, rows, n_out_rows, d, eps);
  }
  dim3 grid(n_out_rows);
  if (d >= 512) {
    if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<bf16, 256>, grid, dim3(256), 0, stream, 1, x, w, (bf16*)out, rows, d, eps);
    return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<float, 256>, grid, dim3(256), 0, stream, 1, x, w, (float*)out, rows, d, eps);
  }
  if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<bf16, 64>, grid, dim3(64), 0, stream, 1, x, w, (bf16*)out, rows, d, eps);
  return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<float, 64>, grid, dim3(64), 0, stream, 1, x, w, (float*)out, rows, d, eps);
}

// ---------------------------------------------------------------- SiLU gate
// in [T, 2F]: gate in columns [0,F), up in [F,2F); out [T,F] = gate/(1+exp(-gate)) * up.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int F) {
  FELLM_TRACE_SCOPE(TRACE_SILU_MUL);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  size_t n = (size_t)rows * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / F; int c = (int)(i - r * F);
    float g = to_f(gu[r * 2 * F + c]);
    float u = to_f(gu[r * 2 * F + F + c]);
    out[i] = from_f<T>((g / (1.0f + expf(-g))) * u);
  }
}

FELLM_API int fellm_silu_mul(const void* gu, void* out, int is_bf16, int rows, int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  size_t n = (size_t)rows * F;
  int blocks = (int)((n + 255) / 256); if (blocks > fellm_sm_count() * 16) blocks = fellm_sm_count() * 16;
  if (is_bf16) return launch_k_class(launch_class_for_rows(rows, 0), silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, (const bf16*)gu, (bf16*)out, rows, F);
  return launch_k_class(launch_class_for_rows(rows, 0), silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (const float*)gu, (float*)out, rows, F);
}

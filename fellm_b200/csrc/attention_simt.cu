// Causal GQA attention over the paged cache on CUDA cores, float32 arithmetic: the engine's
// 32-bit attention, and the yardstick of the tensor-core kernels.
//
// FeLLM counterpart: attention_paged_batch_heads, one thread per (row, head) with a serial
// online softmax over the row's length (plugins/cuda_kernels/src/oxide_kernels.rs:4271-4360;
// formulas crates/fellm-plugin-abi/src/attention_provider.rs:175-237): s_j = (q.k_j)*scale,
// m' = max(m, s), l = l*exp(m-m') + sum exp(s-m'), acc = acc*exp(m-m') + sum p_j v_j, out = acc/l.
//
// One warp per (row, head).  Keys are taken in tiles of 32 that start at the first visible
// position (0, or position-window+1), so the order of every sum depends on the query's position
// alone: not on the cut of the prompt, the batch, or the pages.
#include "common.cuh"

#define MAX_HD 256

template <typename TA, typename TC>
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const TA* __restrict__ q, const TC* __restrict__ pool,
                            const int* __restrict__ block_table, int max_pages,
                            const int* __restrict__ positions, const int* __restrict__ row_slot,
                            TA* __restrict__ out, int T, int H, int G, int hd, int page_tokens, int layer,
                            int layers_in_group, float scale, int window) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_SIMT);
  extern __shared__ float qs_all[];                 // [warps per block][hd]
  int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int warp = blockIdx.x * (blockDim.x >> 5) + wib;
  if (warp >= T * H) return;
  int row = warp / H, h = warp - row * H;
  int g = h / (H / G);
  float* qs = qs_all + (size_t)wib * hd;
  const TA* qr = q + ((size_t)row * H + h) * hd;
  for (int e = lane; e < hd; e += 32) qs[e] = to_f(qr[e]);
  __syncwarp();
  int pos = positions[row];
  const int* bt = block_table + (size_t)row_slot[row] * max_pages;
  int k_begin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int k0 = k_begin; k0 <= pos; k0 += 32) {
    int kj = k0 + lane;
    float s = -INFINITY;
    const TC* vrow = nullptr;
    if (kj <= pos) {
      int page = max(bt[kj / page_tokens], 0);      // an unmapped entry (-1) must never become an address
      size_t base = ((((size_t)page * layers_in_group + layer) * 2) * G + g) * page_tokens + (kj % page_tokens);
      const TC* krow = pool + base * hd;
      vrow = pool + (base + (size_t)G * page_tokens) * hd;
      float dot = 0.f;
      for (int e = 0; e < hd; ++e) dot = fmaf(qs[e], to_f(krow[e]), dot);
      s = dot * scale;
    }
    float m_new = fmaxf(m, warp_max(s));
    float p = kj <= pos ? expf(s - m_new) : 0.f;
    float corr = expf(m - m_new);                  // m = -inf on the first tile: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
    int n_valid = pos - k0 + 1 < 32 ? pos - k0 + 1 : 32;
    for (int j = 0; j < n_valid; ++j) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      const TC* vj = (const TC*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        int e = lane + 32 * i;
        if (e < hd) acc[i] = fmaf(pj, to_f(vj[e]), acc[i]);
      }
    }
  }
  TA* o = out + ((size_t)row * H + h) * hd;
  float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    int e = lane + 32 * i;
    if (e < hd) o[e] = from_f<TA>(acc[i] * inv_l);
  }
}

FELLM_API int fellm_paged_attention_simt(const void* q, int act_bf16, const void* pool, int cache_bf16,
                                         const int* block_table, int max_pages, const int* positions,
                                         const int* row_slot, void* out, int T, int H, int G, int hd,
                                         int page_tokens, int layer, int layers_in_group, float scale,
                                         int window, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd < 1 || hd > MAX_HD) return FELLM_ERR_SIZE;
  if (G < 1 || H % G) return FELLM_ERR_SIZE;
  if (!q || !pool || !block_table || !positions || !row_slot || !out) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  int warps_per_block = 4;
  long long warps = (long long)T * H;
  unsigned blocks = (unsigned)((warps + warps_per_block - 1) / warps_per_block);
  size_t smem = (size_t)warps_per_block * hd * sizeof(float);
  if (act_bf16)
    paged_attention_simt_kernel<bf16, bf16><<<blocks, warps_per_block * 32, smem, stream>>>((const bf16*)q,
        (const bf16*)pool, block_table, max_pages, positions, row_slot, (bf16*)out, T, H, G, hd, page_tokens,
        layer, layers_in_group, scale, window);
  else
    paged_attention_simt_kernel<float, float><<<blocks, warps_per_block * 32, smem, stream>>>((const float*)q,
        (const float*)pool, block_table, max_pages, positions, row_slot, (float*)out, T, H, G, hd, page_tokens,
        layer, layers_in_group, scale, window);
  return launch_status();
}

// Per-head RMSNorm on q and k, rotary position encoding on q and k, and the write of k and v
// into the request's cache pages: one pass over the [T, (H+2G)*hd] output of the QKV product.
//
// FeLLM does this as separate ops: rmsnorm_group (oxide_kernels.rs:165), rope_batch (323),
// kv_write_batch (4227) twice; formulas in crates/backend-cpu/src/kernels/norm.rs:6-39 and
// rope.rs:28-62.  Angle = float32(position) * inv_freq[i]; a' = a*c - b*s, b' = a*s + b*c on
// pairs (2i, 2i+1) (pairing 0, "adjacent") or (i, i+hd/2) (pairing 1, "split_half").
//
// Cache pool layout (one pool per cache group, shared by the group's layers):
//   [page][layer in group][k=0 / v=1][kv head][token in page][hd]
// so that the [page_tokens, hd] tile of one kv head is contiguous.
#include "common.cuh"

template <typename TA, typename TC>
__global__ void qk_rope_write_kernel(const TA* __restrict__ qkv, const float* __restrict__ q_w,
                                     const float* __restrict__ k_w, float eps,
                                     const float* __restrict__ inv_freq, int pairing,
                                     const int* __restrict__ positions, const int* __restrict__ row_slot,
                                     const int* __restrict__ block_table, int max_pages,
                                     TC* __restrict__ pool, int layer, int layers_in_group,
                                     int page_tokens, TA* __restrict__ q_out, int T, int H, int G, int hd,
                                     int write_kv, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  int heads_total = H + 2 * G;
  if (warp >= T * heads_total) return;
  int row = warp / heads_total, head = warp - row * heads_total;
  const TA* src = qkv + (size_t)row * heads_total * hd + (size_t)head * hd;
  int pos = positions[row];
  bool is_q = head < H, is_k = !is_q && head < H + G;
  if (!is_q && !write_kv) return;

  TC* dst_c = nullptr;
  if (!is_q) {
    int g = is_k ? head - H : head - H - G;
    int page = block_table[(size_t)row_slot[row] * max_pages + pos / page_tokens];
    if (page < 0) {                      // never write outside the pool: record and skip
      if (lane == 0 && status) atomicExch(status, 2);
      return;
    }
    size_t off = ((((size_t)page * layers_in_group + layer) * 2 + (is_k ? 0 : 1)) * G + g) * page_tokens
                 + (pos % page_tokens);
    dst_c = pool + off * hd;
  }
  if (!is_q && !is_k) {                  // v: copied as it is
    for (int e = lane; e < hd; e += 32) dst_c[e] = from_f<TC>(to_f(src[e]));
    return;
  }
  const float* nw = is_q ? q_w : k_w;
  int half = hd >> 1;
  float scale = 1.f;
  if (nw) {
    float ss = 0.f;
    for (int e = lane; e < hd; e += 32) { float v = to_f(src[e]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    scale = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  for (int p = lane; p < half; p += 32) {
    int i0 = pairing == 0 ? 2 * p : p;
    int i1 = pairing == 0 ? 2 * p + 1 : p + half;
    float a = to_f(src[i0]), b = to_f(src[i1]);
    if (nw) { a = (a * scale) * nw[i0]; b = (b * scale) * nw[i1]; }
    if (inv_freq) {
      float ang = (float)pos * inv_freq[p];
      float sn, cs;
      sincosf(ang, &sn, &cs);
      float a2 = a * cs - b * sn, b2 = a * sn + b * cs;
      a = a2; b = b2;
    }
    if (is_q) {
      TA* q = q_out + ((size_t)row * H + head) * hd;
      q[i0] = from_f<TA>(a); q[i1] = from_f<TA>(b);
    } else {
      dst_c[i0] = from_f<TC>(a); dst_c[i1] = from_f<TC>(b);
    }
  }
}

FELLM_API int fellm_qk_rope_write(const void* qkv, int act_bf16, const float* q_w, const float* k_w,
                                  float eps, const float* inv_freq, int pairing, const int* positions,
                                  const int* row_slot, const int* block_table, int max_pages, void* pool,
                                  int cache_bf16, int layer, int layers_in_group, int page_tokens,
                                  void* q_out, int T, int H, int G, int hd, int write_kv, int* status,
                                  cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd < 2 || (hd & 1)) return FELLM_ERR_SIZE;
  if (!qkv || !q_out || !positions || !row_slot || (write_kv && (!pool || !block_table))) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  long long warps = (long long)T * (H + 2 * G);
  int threads = 128;
  long long blocks = (warps * 32 + threads - 1) / threads;
  if (act_bf16)
    return launch_k(qk_rope_write_kernel<bf16, bf16>, dim3((unsigned)blocks), dim3(threads), 0, stream, 1,
                    (const bf16*)qkv, q_w, k_w, eps, inv_freq, pairing, positions, row_slot, block_table, max_pages,
                    (bf16*)pool, layer, layers_in_group, page_tokens, (bf16*)q_out, T, H, G, hd, write_kv, status);
  return launch_k(qk_rope_write_kernel<float, float>, dim3((unsigned)blocks), dim3(threads), 0, stream, 1,
                  (const float*)qkv, q_w, k_w, eps, inv_freq, pairing, positions, row_slot, block_table, max_pages,
                  (float*)pool, layer, layers_in_group, page_tokens, (float*)q_out, T, H, G, hd, write_kv, status);
}

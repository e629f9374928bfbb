// Per-head RMSNorm on q and k, rotary position encoding on q and k, and the write of k and v
// into the request's cache pages: one pass over the [T, (H+2G)*hd] output of the QKV product.
//
// FeLLM does this as separate ops: rmsnorm_group (oxide_kernels.rs:165), rope_batch (323),
// kv_write_batch (4227) twice; formulas in crates/backend-cpu/src/kernels/norm.rs:6-39 and
// rope.rs:28-62.  Angle = float32(position) * inv_freq[i]; a' = a*c - b*s, b' = a*s + b*c on
// pairs (2i, 2i+1) (pairing 0, "adjacent") or (i, i+rot_dim/2) (pairing 1, "split_half") of the
// first rot_dim <= hd elements of a head (rope.rs:37-44: rope_dim <= head_dim); the elements
// behind rot_dim are normed and not rotated.  inv_freq has rot_dim/2 entries.
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
                                     int rot_dim, int write_kv, int* __restrict__ status) {
  FELLM_TRACE_SCOPE(TRACE_QK_ROPE_WRITE);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
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
  int half = rot_dim >> 1;
  float scale = 1.f;
  if (nw) {
    float ss = 0.f;
    for (int e = lane; e < hd; e += 32) { float v = to_f(src[e]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    scale = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  for (int e = rot_dim + lane; e < hd; e += 32) {      // behind the rotated part: normed, not rotated
    float a = to_f(src[e]);
    if (nw) a = (a * scale) * nw[e];
    if (is_q) q_out[((size_t)row * H + head) * hd + e] = from_f<TA>(a);
    else dst_c[e] = from_f<TC>(a);
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

// bfloat16, hd % 16 == 0: a head is taken by hd/16 lanes of a group of GL lanes (GL the next power
// of two), each with 16 elements = 8 pairs in two 16-byte loads: elements [16l, 16l+16) when pairs
// are adjacent, [8l, 8l+8) and [hd/2 + 8l, hd/2 + 8l + 8) when they are (i, i + hd/2).
__device__ __forceinline__ void rw_unpack8(uint4 v, float* f) {
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 rw_pack8(const float* f) {
  uint4 v;
  __nv_bfloat162 p0 = __floats2bfloat162_rn(f[0], f[1]), p1 = __floats2bfloat162_rn(f[2], f[3]);
  __nv_bfloat162 p2 = __floats2bfloat162_rn(f[4], f[5]), p3 = __floats2bfloat162_rn(f[6], f[7]);
  v.x = *(unsigned*)&p0; v.y = *(unsigned*)&p1; v.z = *(unsigned*)&p2; v.w = *(unsigned*)&p3;
  return v;
}

template <int GL>
__global__ void qk_rope_write_vec_kernel(const bf16* __restrict__ qkv, const float* __restrict__ q_w,
                                         const float* __restrict__ k_w, float eps,
                                         const float* __restrict__ inv_freq, int pairing,
                                         const int* __restrict__ positions, const int* __restrict__ row_slot,
                                         const int* __restrict__ block_table, int max_pages,
                                         bf16* __restrict__ pool, int layer, int layers_in_group,
                                         int page_tokens, bf16* __restrict__ q_out, int T, int H, int G, int hd,
                                         int write_kv, int* __restrict__ status) {
  FELLM_TRACE_SCOPE(TRACE_QK_ROPE_WRITE_VEC);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / GL;
  const int l = threadIdx.x % GL;
  const int heads_total = H + 2 * G;
  const bool live = gid < (long long)T * heads_total;         // every lane stays for the shuffles
  const int row = live ? (int)(gid / heads_total) : 0, head = live ? (int)(gid - (long long)row * heads_total) : 0;
  const bool is_q = head < H, is_k = !is_q && head < H + G;
  const bool lane_on = live && l * 16 < hd && (is_q || write_kv);
  const int half = hd >> 1;
  const int o0 = pairing == 0 ? 16 * l : 8 * l;               // the lane's two runs of 8 elements
  const int o1 = pairing == 0 ? 16 * l + 8 : half + 8 * l;
  const bf16* src = qkv + ((size_t)row * heads_total + head) * hd;
  const int pos = positions[row];

  bf16* dst = nullptr;
  bool ok = lane_on;
  if (lane_on) {
    if (is_q) dst = q_out + ((size_t)row * H + head) * hd;
    else {
      int g = is_k ? head - H : head - H - G;
      int page = block_table[(size_t)row_slot[row] * max_pages + pos / page_tokens];
      if (page < 0) {                      // never write outside the pool: record and skip
        if (l == 0 && status) atomicExch(status, 2);
        ok = false;
      } else {
        size_t off = ((((size_t)page * layers_in_group + layer) * 2 + (is_k ? 0 : 1)) * G + g) * page_tokens
                     + (pos % page_tokens);
        dst = pool + off * hd;
      }
    }
  }
  uint4 r0 = make_uint4(0, 0, 0, 0), r1 = r0;
  if (lane_on) { r0 = *(const uint4*)(src + o0); r1 = *(const uint4*)(src + o1); }
  const bool is_v = !is_q && !is_k;
  if (is_v) {                              // v: copied as it is; the lanes stay for the warp's shuffles
    if (ok) { *(uint4*)(dst + o0) = r0; *(uint4*)(dst + o1) = r1; }
    ok = false;
  }
  float a[8], b[8];
  rw_unpack8(r0, a); rw_unpack8(r1, b);
  const float* nw = is_q ? q_w : k_w;
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(a[e], a[e], ss);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(b[e], b[e], ss);
#pragma unroll
    for (int o = GL / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
    if (ok) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { a[e] = (a[e] * scale) * nw[o0 + e]; b[e] = (b[e] * scale) * nw[o1 + e]; }
    }
  }
  if (!ok) return;
  if (inv_freq) {
    if (pairing == 0) {                    // pairs (2i, 2i+1): inside each run
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        float sn, cs;
        sincosf((float)pos * inv_freq[(o0 + e) >> 1], &sn, &cs);
        float x = a[e], y = a[e + 1];
        a[e] = x * cs - y * sn; a[e + 1] = x * sn + y * cs;
        sincosf((float)pos * inv_freq[(o1 + e) >> 1], &sn, &cs);
        x = b[e]; y = b[e + 1];
        b[e] = x * cs - y * sn; b[e + 1] = x * sn + y * cs;
      }
    } else {                               // pairs (i, i + hd/2): run a against run b
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float sn, cs;
        sincosf((float)pos * inv_freq[o0 + e], &sn, &cs);
        float x = a[e], y = b[e];
        a[e] = x * cs - y * sn; b[e] = x * sn + y * cs;
      }
    }
  }
  *(uint4*)(dst + o0) = rw_pack8(a);
  *(uint4*)(dst + o1) = rw_pack8(b);
}

FELLM_API int fellm_qk_rope_write(const void* qkv, int act_bf16, const float* q_w, const float* k_w,
                                  float eps, const float* inv_freq, int pairing, const int* positions,
                                  const int* row_slot, const int* block_table, int max_pages, void* pool,
                                  int cache_bf16, int layer, int layers_in_group, int page_tokens,
                                  void* q_out, int T, int H, int G, int hd, int rot_dim, int write_kv,
                                  int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd < 2 || (hd & 1)) return FELLM_ERR_SIZE;
  if (!inv_freq) rot_dim = 0;
  if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return FELLM_ERR_SIZE;
  if (!qkv || !q_out || !positions || !row_slot || (write_kv && (!pool || !block_table))) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  long long warps = (long long)T * (H + 2 * G);
  int threads = 128;
  long long blocks = (warps * 32 + threads - 1) / threads;
  if (act_bf16 && hd % 16 == 0 && hd <= 256 && (rot_dim == hd || rot_dim == 0)) {
    int lanes = hd / 16, gl = 1;
    while (gl < lanes) gl <<= 1;
    long long nthreads = warps * gl;
    dim3 vgrid((unsigned)((nthreads + threads - 1) / threads));
#define RW_VEC(GL_) launch_k_class(launch_class_for_rows(T, 2), qk_rope_write_vec_kernel<GL_>, vgrid, dim3(threads), 0, stream, 1, (const bf16*)qkv, q_w, k_w, \
                             eps, inv_freq, pairing, positions, row_slot, block_table, max_pages, (bf16*)pool, layer,     \
                             layers_in_group, page_tokens, (bf16*)q_out, T, H, G, hd, write_kv, status)
    switch (gl) {
      case 1: return RW_VEC(1);
      case 2: return RW_VEC(2);
      case 4: return RW_VEC(4);
      case 8: return RW_VEC(8);
      default: return RW_VEC(16);
    }
#undef RW_VEC
  }
  if (act_bf16)
    return launch_k_class(launch_class_for_rows(T, 2), qk_rope_write_kernel<bf16, bf16>, dim3((unsigned)blocks), dim3(threads), 0, stream, 1,
                    (const bf16*)qkv, q_w, k_w, eps, inv_freq, pairing, positions, row_slot, block_table, max_pages,
                    (bf16*)pool, layer, layers_in_group, page_tokens, (bf16*)q_out, T, H, G, hd, rot_dim, write_kv, status);
  return launch_k_class(launch_class_for_rows(T, 2), qk_rope_write_kernel<float, float>, dim3((unsigned)blocks), dim3(threads), 0, stream, 1,
                  (const float*)qkv, q_w, k_w, eps, inv_freq, pairing, positions, row_slot, block_table, max_pages,
                  (float*)pool, layer, layers_in_group, page_tokens, (float*)q_out, T, H, G, hd, rot_dim, write_kv, status);
}

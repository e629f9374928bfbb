// One persistent kernel for a whole decode step (every item brings one token, at most 16 items,
// bfloat16): the step's ~90 dependent launches become stages of one cooperative launch, separated
// by a grid barrier (~1 us) instead of a kernel boundary (~4-5 us of launch, fill and drain).
//
// The kernel interprets a program: an array of stage records that the host builds from the
// model's parts (fellm_b200/engine/mega.py).  Stage kinds: embedding gather; skinny product with a
// prologue (RMSNorm of the float32 residual stream | plain bfloat16 rows | the gated short
// convolution computed from the in-projection's output and the request's state) and an epilogue
// (store | add into the residual stream | SiLU(gate)*up | float32 store), optionally preceded by
// a side job that shifts the conv state; QK-norm + rotary + cache write; split-KV attention;
// two-stage argmax.  A part that the program builder does not know keeps the step on the
// per-kernel path.
//
// Weights of the next product stage are requested BEFORE the barrier that ends the current stage,
// so HBM latency hides behind the barrier.  The barrier is a counter in global memory (cooperative
// launch guarantees that all CTAs are resident); its spin is bounded (2 s), after which the CTA
// records code 201 in the status word and goes on, so that a lost CTA cannot hang the GPU.
//
// FeLLM replays its per-op decode step from a CUDA graph (crates/backend-cuda/src/graph.rs:39-160);
// it has no fused step.
#include "attention_mma.cu"        // attend_tile, load_q, tile geometry for -DHD

#define MG_THREADS 256             // one CTA per SM; the inlined product stages want ~250 registers a thread
#define MG_WARPS 8
#define MG_SLOTS 40
#define MG_U 5
#define MG_KCHUNK 32
#define MG_ROWS 16

enum { K_EMBED = 0, K_GEMM = 1, K_ROPE = 2, K_ATTN = 3, K_ARGMAX_PART = 4, K_ARGMAX_FIN = 5 };
enum { E_STORE = 0, E_ACC = 1, E_SWIGLU = 2, E_F32 = 3 };

struct Stage { long long v[MG_SLOTS]; };
#define SP(T, i) ((T)(st.v[i]))
#define SI(i) ((int)st.v[i])
#define SF(i) ((float)__longlong_as_double(st.v[i]))

__device__ __forceinline__ unsigned long long mg_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Grid barrier: one release-add on a counter in global memory per CTA, then one thread polls it
// with acquire loads (cooperative launch guarantees that every CTA is resident).  The spin is
// bounded: after 2 s the CTA records code 201 in the status word and goes on.
__device__ __forceinline__ void grid_barrier(unsigned* counter, unsigned target, int* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(counter) : "memory");
    const unsigned long long t0 = mg_ns();
    unsigned it = 0;
    while (ld_acquire_u32(counter) < target) {
      if ((++it & 1023u) == 0 && mg_ns() - t0 > 2000000000ull) { atomicExch(status, 201); break; }
    }
  }
  __syncthreads();
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 mg_ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// ------------------------------------------------------------------------------------ product stage
// record: 2 x(bf16) 3 xf 4 norm_w 5 eps 6 W 7 bias 8 out 9 epi 10 N 11 K 12 lda 13 ldw 14 ldo
//         15 warps_k 16 k_per_warp 17 xs_stride 18 n_tiles 19 tiles_per_warp
//         20 bcx 21 conv_w 22 conv_b 23 state 24 slot_stride 25 Lc 26 item_slot     (conv prologue)
//         27 upd_bcx 28 upd_state 29 upd_slot_stride 30 upd_Lc 31 upd_d 32 upd_item_slot   (side job)
struct GemmGeom {
  int wn, wk, k_begin, k_len, n_chunks, rounds_per_tile, first_tile, tile_stride, my_tiles, total_rounds;
};
__device__ __forceinline__ GemmGeom gemm_geom(const Stage& st, int warp, int cta, int n_ctas) {
  GemmGeom q;
  const int warps_k = SI(15), k_per_warp = SI(16), K = SI(11), n_tiles = SI(18);
  const int warps_n = MG_WARPS / warps_k;
  q.wn = warp / warps_k; q.wk = warp - q.wn * warps_k;
  q.k_begin = q.wk * k_per_warp;
  q.k_len = max(min(K, q.k_begin + k_per_warp) - q.k_begin, 0);
  q.n_chunks = (q.k_len + MG_KCHUNK - 1) / MG_KCHUNK;
  q.rounds_per_tile = max((q.n_chunks + MG_U - 1) / MG_U, 1);
  q.first_tile = cta * warps_n + q.wn;
  q.tile_stride = n_ctas * warps_n;
  q.my_tiles = q.first_tile < n_tiles ? (n_tiles - q.first_tile + q.tile_stride - 1) / q.tile_stride : 0;
  q.total_rounds = q.my_tiles * q.rounds_per_tile;
  return q;
}
__device__ __forceinline__ void gemm_load_round(const Stage& st, const GemmGeom& q, int r, int lane, uint4* w0, uint4* w1) {
  const int g = lane >> 2, c = lane & 3, N = SI(10), ldw = SI(13);
  int tl = r / q.rounds_per_tile, rr = r - tl * q.rounds_per_tile;
  int n0 = (q.first_tile + tl * q.tile_stride) * MG_ROWS;
  const bf16* W = SP(const bf16*, 6);
  const bf16* p0 = W + (size_t)min(n0 + g, N - 1) * ldw + q.k_begin + c * 8;
  const bf16* p1 = W + (size_t)min(n0 + g + 8, N - 1) * ldw + q.k_begin + c * 8;
#pragma unroll
  for (int u = 0; u < MG_U; ++u) {
    int kk = (rr * MG_U + u) * MG_KCHUNK;
    if (kk + c * 8 < q.k_len) { w0[u] = mg_ldg_stream(p0 + kk); w1[u] = mg_ldg_stream(p1 + kk); }
    else { w0[u] = make_uint4(0, 0, 0, 0); w1[u] = w0[u]; }
  }
}

template <int MT, int EPI>
__device__ __forceinline__ void gemm_epilogue_direct(const Stage& st, float (*acc)[4], int n0, int g, int c) {
  const int M = SI(1), N = SI(10), ldo = SI(14);
  const float* bias = SP(const float*, 7);
  void* out = SP(void*, 8);
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      int m = t * 8 + 2 * c + e;
      if (m >= M) continue;
      if (EPI == E_SWIGLU) {
        int n = n0 + g;
        if (n < N) {
          float gs = acc[t][e], us = acc[t][2 + e];
          if (bias) { gs += bias[n]; us += bias[n + 8]; }
          ((bf16*)out)[(size_t)m * ldo + (n0 >> 1) + g] = __float2bfloat16_rn((gs / (1.0f + expf(-gs))) * us);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          int n = n0 + g + 8 * h;
          if (n >= N) continue;
          float v = acc[t][2 * h + e];
          if (bias) v += bias[n];
          size_t o = (size_t)m * ldo + n;
          if (EPI == E_STORE) ((bf16*)out)[o] = __float2bfloat16_rn(v);
          else if (EPI == E_ACC) ((float*)out)[o] += v;
          else ((float*)out)[o] = v;
        }
      }
    }
  }
}

template <int MT, int EPI>
__device__ void gemm_stage(const Stage& st, unsigned char* smem, float* row_scale, int cta, int n_ctas,
                           uint4* wA0, uint4* wA1, uint4* wB0, uint4* wB1) {
  constexpr int MP = MT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int M = SI(1), N = SI(10), K = SI(11), lda = SI(12), ldo = SI(14), warps_k = SI(15), k_per_warp = SI(16);
  const int xs_stride = SI(17), tiles_per_warp = SI(19);
  const GemmGeom q = gemm_geom(st, warp, cta, n_ctas);

  // ---- side job: shift the conv state of the layer whose out-projection ran in the stage before
  if (st.v[27]) {
    const bf16* ub = SP(const bf16*, 27);
    float* ust = SP(float*, 28);
    const long long ustride = st.v[29];
    const int uLc = SI(30), ud = SI(31), H = uLc - 1;
    const int* uslot = SP(const int*, 32);
    for (int i = cta * MG_THREADS + threadIdx.x; i < M * ud; i += n_ctas * MG_THREADS) {
      int m = i / ud, ch = i - m * ud;
      const bf16* row = ub + (size_t)m * 3 * ud;
      float bx = __bfloat162float(row[ch]) * __bfloat162float(row[2 * ud + ch]);
      float* s = ust + (size_t)uslot[m] * ustride;
      for (int t = 0; t + 1 < H; ++t) s[(size_t)t * ud + ch] = s[(size_t)(t + 1) * ud + ch];
      s[(size_t)(H - 1) * ud + ch] = bx;
    }
  }

  if (cta * (MG_WARPS / warps_k) >= SI(18)) return;      // no slab for this CTA (the same for all its threads)

  // ---- stage x[:, 0:K] as bfloat16 (rows >= M zero)
  bf16* xs = (bf16*)smem;
  const int k_cta = warps_k * k_per_warp, vec_per_row = k_cta / 8;
  const float* xf = SP(const float*, 3);
  const bf16* bcx = SP(const bf16*, 20);
  if (xf) {
    const float* norm_w = SP(const float*, 4);
    const float eps = SF(5);
    for (int r = warp; r < M; r += MG_WARPS) {
      const float4* xr = (const float4*)(xf + (size_t)r * lda);
      float ss = 0.f;
      for (int i = lane; i < K / 4; i += 32) { float4 v = xr[i]; ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss)))); }
      ss = warp_sum(ss);
      if (lane == 0) row_scale[r] = 1.0f / sqrtf(ss / (float)K + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < MT * 8 * vec_per_row; i += MG_THREADS) {
      int r = i / vec_per_row, v = i - r * vec_per_row, k = v * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < M && k < K) {
        const float4* xr = (const float4*)(xf + (size_t)r * lda + k);
        const float4* wr = (const float4*)(norm_w + k);
        float4 x0 = xr[0], x1 = xr[1], g0 = wr[0], g1 = wr[1];
        float sc = row_scale[r];
        val.x = pack_bf16((x0.x * sc) * g0.x, (x0.y * sc) * g0.y); val.y = pack_bf16((x0.z * sc) * g0.z, (x0.w * sc) * g0.w);
        val.z = pack_bf16((x1.x * sc) * g1.x, (x1.y * sc) * g1.y); val.w = pack_bf16((x1.z * sc) * g1.z, (x1.w * sc) * g1.w);
      }
      *(uint4*)(xs + (size_t)r * xs_stride + k) = val;
    }
  } else if (bcx) {
    // y = C * (bx*w[Lc-1] + sum_t state[t]*w[t] + bias), bx = B*X: the decode form of the gated conv
    // (crates/backend-cpu/src/kernels/shortconv.rs:61-106), tap order as in shortconv.cu
    const float* cw = SP(const float*, 21);
    const float* cb = SP(const float*, 22);
    const float* state = SP(const float*, 23);
    const long long sstride = st.v[24];
    const int Lc = SI(25), H = Lc - 1;
    const int* islot = SP(const int*, 26);
    for (int i = threadIdx.x; i < MT * 8 * vec_per_row; i += MG_THREADS) {      // 8 channels a thread
      int r = i / vec_per_row, ch0 = (i - r * vec_per_row) * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < M && ch0 < K) {
        const bf16* row = bcx + (size_t)r * 3 * K;
        float bf_[8], cf_[8], xf_[8], conv[8];
        uint4 bv = *(const uint4*)(row + ch0), cv = *(const uint4*)(row + K + ch0), xv = *(const uint4*)(row + 2 * K + ch0);
        unpack8(bv, bf_); unpack8(cv, cf_); unpack8(xv, xf_);
        const float* s = state + (size_t)islot[r] * sstride;
#pragma unroll
        for (int e = 0; e < 8; ++e) conv[e] = (bf_[e] * xf_[e]) * cw[(size_t)(ch0 + e) * Lc + H];
        for (int t = 0; t < H; ++t) {
          float4 s0 = *(const float4*)(s + (size_t)t * K + ch0), s1 = *(const float4*)(s + (size_t)t * K + ch0 + 4);
          float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) conv[e] = fmaf(sv[e], cw[(size_t)(ch0 + e) * Lc + t], conv[e]);
        }
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = cf_[e] * (conv[e] + (cb ? cb[ch0 + e] : 0.f));
        val.x = pack_bf16(y[0], y[1]); val.y = pack_bf16(y[2], y[3]); val.z = pack_bf16(y[4], y[5]); val.w = pack_bf16(y[6], y[7]);
      }
      *(uint4*)(xs + (size_t)r * xs_stride + ch0) = val;
    }
  } else {
    const bf16* x = SP(const bf16*, 2);
    for (int i = threadIdx.x; i < MT * 8 * vec_per_row; i += MG_THREADS) {
      int r = i / vec_per_row, v = i - r * vec_per_row, k = v * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < M && k < K) val = *(const uint4*)(x + (size_t)r * lda + k);
      *(uint4*)(xs + (size_t)r * xs_stride + k) = val;
    }
  }
  __syncthreads();

  // ---- rounds (the first two were requested before the barrier that opened this stage)
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
  float* slots = (float*)(smem + (size_t)MT * 8 * xs_stride * sizeof(bf16));
  const bf16* xw = xs + (size_t)g * xs_stride + q.k_begin + c * 8;
  const bool direct = warps_k == 1;
  auto compute_round = [&](int r, const uint4* w0, const uint4* w1) {
    int tl = r / q.rounds_per_tile, rr = r - tl * q.rounds_per_tile;
#pragma unroll
    for (int u = 0; u < MG_U; ++u) {
      int ch = rr * MG_U + u;
      if (ch < q.n_chunks) {
        unsigned fa[4] = {w0[u].x, w1[u].x, w0[u].y, w1[u].y};
        unsigned fb[4] = {w0[u].z, w1[u].z, w0[u].w, w1[u].w};
        const bf16* xr = xw + ch * MG_KCHUNK;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          uint4 b = *(const uint4*)(xr + (size_t)t * 8 * xs_stride);
          mma16816(acc[t], fa, b.x, b.y);
          mma16816(acc[t], fb, b.z, b.w);
        }
      }
    }
    if (rr == q.rounds_per_tile - 1) {
      int n0 = (q.first_tile + tl * q.tile_stride) * MG_ROWS;
      if (direct) {
        gemm_epilogue_direct<MT, EPI>(st, acc, n0, g, c);
      } else {
        float* p = slots + ((size_t)warp * tiles_per_warp + tl) * MG_ROWS * MP;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          p[g * MP + t * 8 + 2 * c] = acc[t][0]; p[g * MP + t * 8 + 2 * c + 1] = acc[t][1];
          p[(g + 8) * MP + t * 8 + 2 * c] = acc[t][2]; p[(g + 8) * MP + t * 8 + 2 * c + 1] = acc[t][3];
        }
      }
#pragma unroll
      for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
    }
  };
  for (int r = 0; r < q.total_rounds; r += 2) {
    compute_round(r, wA0, wA1);
    if (r + 2 < q.total_rounds) gemm_load_round(st, q, r + 2, lane, wA0, wA1);
    if (r + 1 < q.total_rounds) {
      compute_round(r + 1, wB0, wB1);
      if (r + 3 < q.total_rounds) gemm_load_round(st, q, r + 3, lane, wB0, wB1);
    }
  }
  if (direct) return;
  __syncthreads();
  // ---- sum the K warps' partial slabs in warp order; every K warp finishes a share of the rows
  const float* bias = SP(const float*, 7);
  void* out = SP(void*, 8);
  const float* slab_slots = slots + (size_t)(q.wn * warps_k) * tiles_per_warp * MG_ROWS * MP;
  const size_t warp_stride = (size_t)tiles_per_warp * MG_ROWS * MP;
  for (int tl = 0; tl < q.my_tiles; ++tl) {
    int n0 = (q.first_tile + tl * q.tile_stride) * MG_ROWS;
    const float* mine = slab_slots + (size_t)tl * MG_ROWS * MP;
    const int units = (EPI == E_SWIGLU ? 8 : MG_ROWS) * M;
    for (int i = q.wk * 32 + lane; i < units; i += warps_k * 32) {
      int m, j;
      if (EPI == E_SWIGLU) { m = i >> 3; j = i & 7; } else { m = i >> 4; j = i & 15; }
      float v0 = 0.f, v1 = 0.f;
      for (int w = 0; w < warps_k; ++w) {
        v0 += mine[w * warp_stride + j * MP + m];
        if (EPI == E_SWIGLU) v1 += mine[w * warp_stride + (j + 8) * MP + m];
      }
      int n = n0 + j;
      if (n >= N) continue;
      if (EPI == E_SWIGLU) {
        if (bias) { v0 += bias[n]; v1 += bias[n + 8]; }
        ((bf16*)out)[(size_t)m * ldo + (n0 >> 1) + j] = __float2bfloat16_rn((v0 / (1.0f + expf(-v0))) * v1);
      } else {
        if (bias) v0 += bias[n];
        size_t o = (size_t)m * ldo + n;
        if (EPI == E_STORE) ((bf16*)out)[o] = __float2bfloat16_rn(v0);
        else if (EPI == E_ACC) ((float*)out)[o] += v0;
        else ((float*)out)[o] = v0;
      }
    }
  }
}

__device__ void gemm_dispatch(const Stage& st, unsigned char* smem, float* row_scale, int cta, int n_ctas,
                              uint4* wA0, uint4* wA1, uint4* wB0, uint4* wB1) {
  const int epi = SI(9), mt2 = SI(1) > 8;
#define MG_CASE(E) if (mt2) gemm_stage<2, E>(st, smem, row_scale, cta, n_ctas, wA0, wA1, wB0, wB1); \
                   else gemm_stage<1, E>(st, smem, row_scale, cta, n_ctas, wA0, wA1, wB0, wB1);
  if (epi == E_STORE) { MG_CASE(E_STORE) } else if (epi == E_ACC) { MG_CASE(E_ACC) }
  else if (epi == E_SWIGLU) { MG_CASE(E_SWIGLU) } else { MG_CASE(E_F32) }
#undef MG_CASE
}

// ------------------------------------------------------------------------------------ small stages
// embed: 2 tokens 3 table(bf16) 4 out(f32) 5 d 6 vocab 7 status
__device__ __noinline__ void embed_stage(const Stage& st, int cta, int n_ctas) {
  const int M = SI(1), d = SI(5), vocab = SI(6);
  const int* tokens = SP(const int*, 2);
  const bf16* table = SP(const bf16*, 3);
  float* out = SP(float*, 4);
  for (int i = cta * MG_THREADS + threadIdx.x; i < M * d; i += n_ctas * MG_THREADS) {
    int m = i / d, k = i - m * d, tok = tokens[m];
    float v = 0.f;
    if (tok >= 0 && tok < vocab) v = __bfloat162float(table[(size_t)tok * d + k]);
    else if (k == 0) atomicExch(SP(int*, 7), 1);
    out[i] = v;
  }
}
// rope: 2 qkv 3 q_w 4 k_w 5 eps 6 inv_freq 7 pairing 8 positions 9 row_slot 10 block_table 11 max_pages
//       12 pool 13 layer 14 layers_in_group 15 page_tokens 16 q_out 17 H 18 G 19 status
__device__ __noinline__ void rope_stage(const Stage& st, int cta, int n_ctas) {
  const int M = SI(1), H = SI(17), G = SI(18), heads_total = H + 2 * G;
  const int warp_g = cta * MG_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const bf16* qkv = SP(const bf16*, 2);
  const float* q_w = SP(const float*, 3);
  const float* k_w = SP(const float*, 4);
  const float eps = SF(5);
  const float* inv_freq = SP(const float*, 6);
  const int pairing = SI(7), max_pages = SI(11), layer = SI(13), lig = SI(14), pt = SI(15);
  const int* positions = SP(const int*, 8);
  const int* row_slot = SP(const int*, 9);
  const int* block_table = SP(const int*, 10);
  bf16* pool = SP(bf16*, 12);
  bf16* q_out = SP(bf16*, 16);
  for (int job = warp_g; job < M * heads_total; job += n_ctas * MG_WARPS) {
    int row = job / heads_total, head = job - row * heads_total;
    const bf16* src = qkv + (size_t)row * heads_total * HD + (size_t)head * HD;
    int pos = positions[row];
    bool is_q = head < H, is_k = !is_q && head < H + G;
    bf16* dst = nullptr;
    if (!is_q) {
      int g = is_k ? head - H : head - H - G;
      int page = block_table[(size_t)row_slot[row] * max_pages + pos / pt];
      if (page < 0) { if (lane == 0) atomicExch(SP(int*, 19), 2); continue; }
      size_t off = ((((size_t)page * lig + layer) * 2 + (is_k ? 0 : 1)) * G + g) * pt + (pos % pt);
      dst = pool + off * HD;
    }
    if (!is_q && !is_k) { for (int e = lane; e < HD; e += 32) dst[e] = src[e]; continue; }
    const float* nw = is_q ? q_w : k_w;
    float scale = 1.f;
    if (nw) {
      float ss = 0.f;
      for (int e = lane; e < HD; e += 32) { float v = __bfloat162float(src[e]); ss = fmaf(v, v, ss); }
      ss = warp_sum(ss);
      scale = 1.0f / sqrtf(ss / (float)HD + eps);
    }
    for (int p = lane; p < HD / 2; p += 32) {
      int i0 = pairing == 0 ? 2 * p : p, i1 = pairing == 0 ? 2 * p + 1 : p + HD / 2;
      float a = __bfloat162float(src[i0]), b = __bfloat162float(src[i1]);
      if (nw) { a = (a * scale) * nw[i0]; b = (b * scale) * nw[i1]; }
      if (inv_freq) {
        float sn, cs;
        sincosf((float)pos * inv_freq[p], &sn, &cs);
        float a2 = a * cs - b * sn, b2 = a * sn + b * cs;
        a = a2; b = b2;
      }
      bf16* o = is_q ? q_out + ((size_t)row * H + head) * HD : dst;
      o[i0] = __float2bfloat16_rn(a); o[i1] = __float2bfloat16_rn(b);
    }
  }
}

// attention: 2 q 3 pool 4 block_table 5 max_pages 6 positions 7 row_slot 8 out 9 scratch 10 counters
//            11 H 12 G 13 page_tokens 14 layer 15 layers_in_group 16 scale_log2 17 window 18 split_len 19 max_splits
constexpr int MG_RING = DC_WARPS * DC_STAGES * 2 * DC_TK * ROWB;          // bytes of one virtual CTA's rings
constexpr int MG_VCTAS = (2 * MG_RING <= 196 * 1024) ? 2 : 1;           // virtual CTAs of 4 warps in the 8-warp CTA
__device__ __forceinline__ void vcta_sync(int vc) { asm volatile("bar.sync %0, 128;\n" ::"r"(vc + 1) : "memory"); }

__device__ __noinline__ void attn_stage(const Stage& st, unsigned char* smem_all, int* sm_pages_all, int* sm_last_all, int cta, int n_ctas) {
  const int vc = threadIdx.x >> 7;                      // virtual CTA of 4 warps
  if (vc >= MG_VCTAS) return;
  const int tid = threadIdx.x & 127, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, c = lane & 3;
  unsigned char* smem = smem_all + (size_t)vc * MG_RING;
  int* sm_pages = sm_pages_all + vc * DC_MAX_PAGES;
  int* sm_last = sm_last_all + vc;
  const int M = SI(1), H = SI(11), G = SI(12), pt = SI(13), layer = SI(14), lig = SI(15), window = SI(17);
  const int split_len = SI(18), max_splits = SI(19), max_pages = SI(5), R = H / G;
  const float scale_log2 = SF(16);
  const bf16* qp = SP(const bf16*, 2);
  const bf16* pool = SP(const bf16*, 3);
  const int* block_table = SP(const int*, 4);
  const int* positions = SP(const int*, 6);
  const int* row_slot = SP(const int*, 7);
  bf16* out = SP(bf16*, 8);
  float* scratch = SP(float*, 9);
  int* counters = SP(int*, 10);
  constexpr int TILE_B = DC_TK * ROWB;
  constexpr int SW = HD + 2;
  const size_t page_elems = (size_t)pt * HD;
  const int total = max_splits * G * M;
  for (int vb = cta * MG_VCTAS + vc; vb < total; vb += n_ctas * MG_VCTAS) {
    const int s = vb % max_splits, g = (vb / max_splits) % G, t = vb / (max_splits * G);
    const int pos = positions[t];
    const int kb = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int s_lo = kb / split_len, s_hi = pos / split_len;
    if (s < s_lo || s > s_hi) continue;                 // uniform over the virtual CTA
    const int n_active = s_hi - s_lo + 1;
    const int k0 = max(kb, s * split_len), k1 = min(pos + 1, (s + 1) * split_len);
    const int* bt = block_table + (size_t)row_slot[t] * max_pages;
    const int pg0 = k0 / pt, n_pg = (k1 - 1) / pt - pg0 + 1;
    const bool pages_in_smem = n_pg <= DC_MAX_PAGES;
    vcta_sync(vc);                                      // the previous unit is done with smem
    if (pages_in_smem)
      for (int i = tid; i < n_pg; i += 128) sm_pages[i] = bt[pg0 + i];
    vcta_sync(vc);
    const unsigned ring = (unsigned)__cvta_generic_to_shared(smem) + warp * DC_STAGES * 2 * TILE_B;
    float* merge = (float*)smem;
    const int cta_step = DC_WARPS * DC_TK;
    const int n_tiles = (k1 - k0 - warp * DC_TK + cta_step - 1) / cta_step;
    auto issue = [&](int j) {
      if (j < n_tiles) {
        unsigned ks = ring + (j % DC_STAGES) * 2 * TILE_B, vs = ks + TILE_B;
        int key0 = k0 + (j * DC_WARPS + warp) * DC_TK;
        for (int i = lane; i < DC_TK * CPR; i += 32) {
          int row = i / CPR, ch = i - row * CPR, key = key0 + row;
          if (key < k1) {
            int lp = key / pt;
            int page = pages_in_smem ? sm_pages[lp - pg0] : bt[lp];
            const bf16* kp = pool + ((((size_t)page * lig + layer) * 2) * G + g) * page_elems + (size_t)(key - lp * pt) * HD + ch * 8;
            cp_async16(ks + tile_off(row, ch), kp);
            cp_async16(vs + tile_off(row, ch), kp + (size_t)G * page_elems);
          } else {
            st_shared_zero16(ks + tile_off(row, ch));
            st_shared_zero16(vs + tile_off(row, ch));
          }
        }
      }
      cp_async_commit();
    };
    for (int r0 = 0; r0 < R; r0 += 16) {
#pragma unroll
      for (int j = 0; j < DC_STAGES - 1; ++j) issue(j);
      unsigned qf[KS][4];
      load_q(qf, [&](int i) -> const bf16* { return r0 + i < R ? qp + ((size_t)t * H + g * R + r0 + i) * HD : nullptr; }, lane);
      float o[DN][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
      for (int d = 0; d < DN; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
      int lo[2] = {k0, k0}, hi[2] = {k1 - 1, k1 - 1};
      for (int j = 0; j < n_tiles; ++j) {
        issue(j + DC_STAGES - 1);
        cp_async_wait<DC_STAGES - 1>();
        __syncwarp();
        unsigned ks = ring + (j % DC_STAGES) * 2 * TILE_B, vs = ks + TILE_B;
        attend_tile<DC_TK / 8>(qf, ks, vs, k0 + (j * DC_WARPS + warp) * DC_TK, lo, hi, scale_log2, o, m, l, lane);
        __syncwarp();
      }
      cp_async_wait<0>();
      vcta_sync(vc);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        float* rec = merge + ((size_t)warp * 16 + gq + 8 * r) * SW;
#pragma unroll
        for (int d = 0; d < DN; ++d) { rec[d * 8 + 2 * c] = o[d][2 * r]; rec[d * 8 + 2 * c + 1] = o[d][2 * r + 1]; }
        if (c == 0) { rec[HD] = m[r]; rec[HD + 1] = l[r]; }
      }
      vcta_sync(vc);
      const int rows_here = min(16, R - r0);
      for (int i = tid; i < rows_here * HD; i += 128) {
        int row = i / HD, d = i - row * HD;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) mx = fmaxf(mx, merge[((size_t)w * 16 + row) * SW + HD]);
        float lt = 0.f, at = 0.f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) {
          const float* rec = merge + ((size_t)w * 16 + row) * SW;
          float cw = rec[HD] == -INFINITY ? 0.f : exp2f(rec[HD] - mx);
          lt += rec[HD + 1] * cw;
          at += rec[d] * cw;
        }
        int h = g * R + r0 + row;
        if (n_active == 1) out[((size_t)t * H + h) * HD + d] = __float2bfloat16_rn(at / lt);
        else {
          float* rec = scratch + (((size_t)t * H + h) * max_splits + (s - s_lo)) * SW;
          rec[d] = at;
          if (d == 0) { rec[HD] = mx; rec[HD + 1] = lt; }
        }
      }
      vcta_sync(vc);
    }
    if (n_active == 1) continue;
    __threadfence();
    vcta_sync(vc);
    if (tid == 0) {
      int old = atomicAdd(&counters[t * G + g], 1);
      *sm_last = (old == n_active - 1);
      if (*sm_last) counters[t * G + g] = 0;
    }
    vcta_sync(vc);
    if (!*sm_last) continue;
    __threadfence();
    for (int i = tid; i < R * HD; i += 128) {
      int r = i / HD, d = i - r * HD, h = g * R + r;
      const float* rec = scratch + ((size_t)t * H + h) * max_splits * SW;
      float mx = -INFINITY;
      for (int j = 0; j < n_active; ++j) mx = fmaxf(mx, rec[(size_t)j * SW + HD]);
      float lt = 0.f, at = 0.f;
      for (int j = 0; j < n_active; ++j) {
        float cj = exp2f(rec[(size_t)j * SW + HD] - mx);
        lt += rec[(size_t)j * SW + HD + 1] * cj;
        at += rec[(size_t)j * SW + d] * cj;
      }
      out[((size_t)t * H + h) * HD + d] = __float2bfloat16_rn(at / lt);
    }
  }
}

// argmax: 2 logits 3 V 4 pval 5 pidx 6 out_tokens; 64 chunks per row, ties to the lower id
#define MG_ARG_CHUNKS 64
__device__ __noinline__ void argmax_part_stage(const Stage& st, float* sb, int* si, int cta, int n_ctas) {
  const int M = SI(1), V = SI(3);
  const float* logits = SP(const float*, 2);
  float* pval = SP(float*, 4);
  int* pidx = SP(int*, 5);
  const int per = (V + MG_ARG_CHUNKS - 1) / MG_ARG_CHUNKS;
  for (int job = cta; job < M * MG_ARG_CHUNKS; job += n_ctas) {
    int row = job / MG_ARG_CHUNKS, chunk = job - row * MG_ARG_CHUNKS;
    int lo = chunk * per, hi = min(V, lo + per);
    const float* lg = logits + (size_t)row * V;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int v = lo + threadIdx.x; v < hi; v += MG_THREADS) { float x = lg[v]; if (x > best) { best = x; bi = v; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < MG_WARPS; ++w) if (sb[w] > best || (sb[w] == best && si[w] < bi)) { best = sb[w]; bi = si[w]; }
      pval[job] = best; pidx[job] = bi;
    }
  }
}
__device__ __noinline__ void argmax_fin_stage(const Stage& st, int cta, int n_ctas) {
  const int M = SI(1);
  const float* pval = SP(const float*, 4);
  const int* pidx = SP(const int*, 5);
  int* out_tokens = SP(int*, 6);
  const int warp_g = cta * MG_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  for (int row = warp_g; row < M; row += n_ctas * MG_WARPS) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int cc = lane; cc < MG_ARG_CHUNKS; cc += 32) {
      float x = pval[row * MG_ARG_CHUNKS + cc]; int i = pidx[row * MG_ARG_CHUNKS + cc];
      if (x > best || (x == best && i < bi)) { best = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) out_tokens[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

// ------------------------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(MG_THREADS, 1)
decode_mega_kernel(const Stage* __restrict__ program, int n_stages, unsigned* barrier, int* status,
                   unsigned long long* trace) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float row_scale[16];
  __shared__ int sm_pages[4 * DC_MAX_PAGES];
  __shared__ int sm_last[4];
  __shared__ float sb[MG_WARPS];
  __shared__ int si[MG_WARPS];
  __shared__ Stage sbuf[2];                               // this stage's record and the next one's
  const int cta = blockIdx.x, n_ctas = gridDim.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint4 wA0[MG_U], wA1[MG_U], wB0[MG_U], wB1[MG_U];
  bool have = false;
  if (threadIdx.x < MG_SLOTS) sbuf[0].v[threadIdx.x] = program[0].v[threadIdx.x];
  __syncthreads();
  for (int i = 0; i < n_stages; ++i) {
    const Stage& st = sbuf[i & 1];
    // the next record travels while this stage runs
    long long next_field = 0;
    if (i + 1 < n_stages && threadIdx.x < MG_SLOTS) next_field = program[i + 1].v[threadIdx.x];
    if (trace && cta == 0 && threadIdx.x == 0) trace[2 * i] = mg_ns();            // stage opens (CTA 0's clock)
    const int kind = SI(0);
    if (kind == K_GEMM) {
      if (!have) {
        GemmGeom q = gemm_geom(st, warp, cta, n_ctas);
        if (q.total_rounds > 0) gemm_load_round(st, q, 0, lane, wA0, wA1);
        if (q.total_rounds > 1) gemm_load_round(st, q, 1, lane, wB0, wB1);
      }
      gemm_dispatch(st, smem, row_scale, cta, n_ctas, wA0, wA1, wB0, wB1);
    } else if (kind == K_EMBED) embed_stage(st, cta, n_ctas);
    else if (kind == K_ROPE) rope_stage(st, cta, n_ctas);
    else if (kind == K_ATTN) attn_stage(st, smem, sm_pages, sm_last, cta, n_ctas);
    else if (kind == K_ARGMAX_PART) argmax_part_stage(st, sb, si, cta, n_ctas);
    else if (kind == K_ARGMAX_FIN) argmax_fin_stage(st, cta, n_ctas);
    have = false;
    if (trace && cta == 0) { __syncthreads(); if (threadIdx.x == 0) trace[2 * i + 1] = mg_ns(); }   // CTA 0 is done with it
    if (i + 1 < n_stages) {
      if (threadIdx.x < MG_SLOTS) sbuf[(i + 1) & 1].v[threadIdx.x] = next_field;
      __syncthreads();
      // weights of the next product: requested now, landed by the time the barrier opens
      const Stage& nx = sbuf[(i + 1) & 1];
      if ((int)nx.v[0] == K_GEMM) {
        GemmGeom q = gemm_geom(nx, warp, cta, n_ctas);
        if (q.total_rounds > 0) gemm_load_round(nx, q, 0, lane, wA0, wA1);
        if (q.total_rounds > 1) gemm_load_round(nx, q, 1, lane, wB0, wB1);
        have = true;
      }
      grid_barrier(barrier, (unsigned)(i + 1) * (unsigned)n_ctas, status);
    }
  }
}

FELLM_API int fellm_decode_mega_smem(int max_x_bytes) {
  int attn = MG_VCTAS * MG_RING;
  return attn > max_x_bytes ? attn : max_x_bytes;
}
FELLM_API int fellm_decode_mega_slots() { return MG_SLOTS; }

// program: n_stages records of MG_SLOTS 8-byte fields on the device; barrier: one uint32 (cleared
// here); smem_bytes: fellm_decode_mega_smem(the largest staged x + slab slots of the program).
// trace: null, or 2*n_stages uint64 that receive, from CTA 0, the time (ns) each stage opened and the time
// CTA 0 finished its share of it.
FELLM_API int fellm_decode_mega(const void* program, int n_stages, unsigned* barrier, int* status, int smem_bytes,
                                unsigned long long* trace, cudaStream_t stream) {
  if (n_stages <= 0) return 0;
  if (!program || !barrier || !status) return FELLM_ERR_ARG;
  if (smem_bytes > 220 * 1024) return FELLM_ERR_SIZE;
  static int n_sm = 0, ready_smem = -1;
  cudaError_t e;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    e = cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
  }
  if (smem_bytes > ready_smem) {
    e = cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel, MG_THREADS, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return FELLM_ERR_SIZE;
    ready_smem = smem_bytes;
  }
  e = cudaMemsetAsync(barrier, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) return (int)e;
  const Stage* prog = (const Stage*)program;
  void* args[] = {(void*)&prog, (void*)&n_stages, (void*)&barrier, (void*)&status, (void*)&trace};
  e = cudaLaunchCooperativeKernel((void*)decode_mega_kernel, dim3(n_sm), dim3(MG_THREADS), args, (size_t)smem_bytes, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

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

#define FELLM_WEIGHT_PREFETCH 1
#include "common.cuh"
namespace cg = cooperative_groups;

#define SK_ROWS 16
#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define KCHUNK 32
#define SK_U 5                       // chunks per round: 10 x 16 B per thread, two rounds in flight
#define SK_XF 2048                   // floats of a row that a warp's float32 buffer takes at a time
#define SK_GAMMA_MAX 2048            // norm weights of up to this many columns are parked in shared memory

enum { EPI_STORE = 0, EPI_ACC = 1, EPI_SWIGLU = 2, EPI_F32 = 3, EPI_CONV = 4, EPI_ARGMAX = 5 };
#define SK_MAX_LC 8

__device__ __forceinline__ void mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void sk_cp_async16(unsigned smem_addr, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem));
}
__device__ __forceinline__ void sk_cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

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
  int M, N, K, lda, ldw, ldo, k_per_cta, xs_stride, splits, warps_k, n_tiles, tiles_per_warp, gamma_offset, xf_offset,
      log2_warps_k, k_per_warp, pdl, chunks_per_warp;
  // EPI_CONV: the gated short convolution behind the input product of a ShortConv mixer
  const float* conv_w; const float* conv_bias; float* conv_state; const int* row_slot;
  long long conv_slot_stride; int conv_taps, red_offset;
  const void* next_w; long long next_bytes;     // the next product's weights, asked into L2 (or null)
  // EPI_ARGMAX: nothing of [M, N] is stored; every CTA leaves its best (value, index) of each row as a key
  // in arg_keys[row * CTAs + CTA] (larger key = larger value, then lower index)
  unsigned long long* arg_keys;
  // EPI_ACC as the producer of the next RMSNorm's input (nn_x null: not asked for): beside out += ..., the
  // single-shot kernel leaves nn_x[m, n] = bfloat16(out[m, n] * nn_w[n]) and, for every slab of 16 columns,
  // nn_ssq[m * n_tiles + slab] = the sum of out[m, n]^2 over the slab
  const float* nn_w; bf16* nn_x; float* nn_ssq; int nn_ldx;
  // ... and its consumer (rs_ssq null: none): x is such an nn_x, and every finished sum of row m is
  // multiplied by 1 / sqrt(sum_p rs_ssq[m * rs_parts + p] / K + rs_eps) before the bias is added:
  // RMSNorm(x) W^T with the row's factor taken out of the product
  const float* rs_ssq; int rs_parts; float rs_eps;
};

// What the next call of this module is to hand on or to take over (see SkinnyArgs); every entry point
// takes it and clears it.
struct NormHandoff { const float* nn_w; void* nn_x; float* nn_ssq; int nn_ldx; const float* rs_ssq; int rs_parts; float rs_eps; };
static NormHandoff g_handoff = {nullptr, nullptr, nullptr, 0, nullptr, 0, 0.f};
static inline NormHandoff take_handoff() {
  NormHandoff h = g_handoff;
  g_handoff = NormHandoff{nullptr, nullptr, nullptr, 0, nullptr, 0, 0.f};
  return h;
}

// float32 value and index as one number whose order is "the larger value, then the lower index":
// greedy sampling's rule (crates/fellm-runtime/src/sampling.rs:588-604).
__device__ __forceinline__ unsigned long long argmax_key(float v, int n) {
  v += 0.0f;                                             // -0 counts as +0
  unsigned u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)n);
}

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

// One row of 128*J floats from the warp's piece: RMSNorm in the order of the general path (lane l
// sums the float4s l, l+32, ... in turn), written as bfloat16.
template <int J>
__device__ __forceinline__ void norm_row_fast(const float4* piece, const float4* gamma_s, bf16* row, int lane, int K, float eps) {
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const float4 v = piece[lane + 32 * j];
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
  }
  ss = warp_sum(ss);
  const float sc = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
  for (int j = 0; j < J; ++j) {                      // read again from shared memory: cheaper than 4*J registers
    const float4 v = piece[lane + 32 * j], gw = gamma_s[lane + 32 * j];
    __nv_bfloat162 p0 = __floats2bfloat162_rn((v.x * sc) * gw.x, (v.y * sc) * gw.y);
    __nv_bfloat162 p1 = __floats2bfloat162_rn((v.z * sc) * gw.z, (v.w * sc) * gw.w);
    uint2 val; val.x = *(unsigned*)&p0; val.y = *(unsigned*)&p1;
    *(uint2*)(row + 4 * (lane + 32 * j)) = val;
  }
}

// MT: token tiles of 8 (M <= 8*MT).
template <int MT, int EPI>
__global__ void __launch_bounds__(SK_THREADS, MT <= 2 ? 2 : 1) gemm_skinny_kernel(SkinnyArgs a) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_SKINNY + 32 * EPI);
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int MP = MT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = a.splits > 1 ? (int)cg::this_cluster().block_rank() : 0;
  // the CTA's warps: wn = which slab of the CTA's pass, wk = which slice of the CTA's K range
  // (warps_k is a power of two; no division by a run-time value on the way to the first load)
  const int warps_n = SK_WARPS >> a.log2_warps_k;
  const int wn = warp >> a.log2_warps_k, wk = warp & (a.warps_k - 1);
  const int k_cta = split * a.k_per_cta;
  const int k_begin = k_cta + wk * a.k_per_warp;                     // k_per_warp: a multiple of 32
  const int k_len = max(min(a.K, k_begin + a.k_per_warp) - k_begin, 0);
  const int n_chunks = (k_len + KCHUNK - 1) / KCHUNK;
  const int rounds_per_tile = max((n_chunks + SK_U - 1) / SK_U, 1);
  // this warp's slabs: first_tile, first_tile + tile_stride, ...: tiles_per_warp of them, or one less
  const int first_tile = blockIdx.y * warps_n + wn;
  const int tile_stride = gridDim.y * warps_n;
  const int my_tiles = first_tile >= a.n_tiles ? 0
                       : a.tiles_per_warp - (first_tile + (a.tiles_per_warp - 1) * tile_stride >= a.n_tiles ? 1 : 0);
  const int total_rounds = my_tiles * rounds_per_tile;
  auto advance = [&](int& tl, int& rr) { if (++rr == rounds_per_tile) { rr = 0; ++tl; } };

  // a round is SK_U chunks of 32 k; all of them whole (the common case) means no test per load
  const bool ragged = (k_len & (KCHUNK - 1)) != 0;                   // the last chunk stops inside its 32 k
  auto load_round = [&](int tl, int rr, uint4* w0, uint4* w1) {
    const int n0 = (first_tile + tl * tile_stride) * SK_ROWS;
    const int k0 = k_begin + c * 8 + rr * (SK_U * KCHUNK);
    const bf16* p0 = a.W + (size_t)min(n0 + g, a.N - 1) * a.ldw + k0;      // rows past N: clamped, never stored
    const bf16* p1 = a.W + (size_t)min(n0 + g + 8, a.N - 1) * a.ldw + k0;
    const int n_valid = n_chunks - rr * SK_U;                        // chunks of this round, warp-uniform
    if (n_valid >= SK_U && !ragged) {
#pragma unroll
      for (int u = 0; u < SK_U; ++u) { w0[u] = ldg_stream(p0 + u * KCHUNK); w1[u] = ldg_stream(p1 + u * KCHUNK); }
    } else {
      const int rem = k_len - rr * (SK_U * KCHUNK) - c * 8;          // this thread's 8 k of chunk u exist if u*32 < rem
#pragma unroll
      for (int u = 0; u < SK_U; ++u) {
        if (u * KCHUNK < rem) { w0[u] = ldg_stream(p0 + u * KCHUNK); w1[u] = ldg_stream(p1 + u * KCHUNK); }
        else { w0[u] = make_uint4(0, 0, 0, 0); w1[u] = w0[u]; }
      }
    }
  };

  // ---- x[:, k_cta : k_cta + k_per_cta] goes to shared memory as bfloat16 (rows >= M zero), normed
  // if asked.  All of it is requested with cp.async before any of it is used: a chain of dependent
  // round trips to L2 is what a step of a few rows would otherwise spend most of its time on.
  bf16* xs = (bf16*)smem;
  const int vec_per_row = a.k_per_cta >> 3;
  const int nv = a.K >> 2;                                           // float4s of a float32 row
  const bool gamma_staged = a.xf && a.K <= SK_GAMMA_MAX;
  float4* piece = (float4*)(smem + a.xf_offset) + (size_t)warp * (min(a.K, SK_XF) / 4);   // the warp's float32 row piece
  const unsigned piece_s = (unsigned)__cvta_generic_to_shared(piece);
  auto request_piece = [&](const float* xrow, int pc) {
    const int v0 = pc * (SK_XF / 4), v1 = min(nv, v0 + SK_XF / 4);
    for (int i = v0 + lane; i < v1; i += 32) sk_cp_async16(piece_s + 16u * (i - v0), xrow + 4 * i);
  };
  auto request_x = [&]() {
    if (a.xf) {
      if (warp < a.M) request_piece(a.xf + (size_t)warp * a.lda, 0);
    } else {
      const unsigned xs_s = (unsigned)__cvta_generic_to_shared(xs);
      const int live_vec = min(vec_per_row, max(a.K - k_cta, 0) >> 3);      // K % 8 == 0: whole vectors
      for (int r = warp; r < MP; r += SK_WARPS) {
        bf16* dst = xs + (size_t)r * a.xs_stride;
        if (r < a.M) {
          const bf16* src = a.x + (size_t)r * a.lda + k_cta;
          const unsigned dst_s = xs_s + 2u * (unsigned)(r * a.xs_stride);
          for (int vv = lane; vv < live_vec; vv += 32) sk_cp_async16(dst_s + 16u * vv, src + vv * 8);
          for (int vv = live_vec + lane; vv < vec_per_row; vv += 32) *(uint4*)(dst + vv * 8) = make_uint4(0, 0, 0, 0);
        } else {
          for (int vv = lane; vv < vec_per_row; vv += 32) *(uint4*)(dst + vv * 8) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  };

  // ---- requests.  The norm's weights and W are parameters: they never wait for the kernel before
  // this one.  As a programmatic dependent the kernel asks for W, waits, then asks for x; launched
  // the ordinary way it asks for the few KB of x first, so that they do not queue behind W.
  if (gamma_staged) {
    const unsigned gs = (unsigned)__cvta_generic_to_shared(smem + a.gamma_offset);
    for (int i = threadIdx.x; i < nv; i += SK_THREADS) sk_cp_async16(gs + 16u * i, a.norm_w + 4 * i);
  }
  if (!a.pdl) request_x();
  uint4 wA0[SK_U], wA1[SK_U], wB0[SK_U], wB1[SK_U];
  int ltl = 0, lrr = 0;
  if (total_rounds > 0) { load_round(ltl, lrr, wA0, wA1); advance(ltl, lrr); }
  if (total_rounds > 1) { load_round(ltl, lrr, wB0, wB1); advance(ltl, lrr); }
  if (threadIdx.x < 32)                                   // (a lane a piece: one thread's loop was 40 turns long for a wide matrix)
    l2_prefetch_share(a.next_w, a.next_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, gridDim.x * gridDim.y * gridDim.z, lane, 32);
  pdl_launch_dependents();
  if (a.pdl) {
    pdl_wait();
    request_x();
  }
  FELLM_TRACE_WAITED();

  if (a.xf) {
    // RMSNorm (crates/backend-cpu/src/kernels/norm.rs:6-39) over the whole row, whatever the slice:
    // a warp per row; the row goes through the warp's float32 buffer in pieces of SK_XF floats, lane
    // l taking the float4s l, l+32, ... of each piece (one piece, read once, when K <= SK_XF)
    const float4* wr = (const float4*)a.norm_w;
    const float4* gamma_s = (const float4*)(smem + a.gamma_offset);
    const int n_pieces = (nv + SK_XF / 4 - 1) / (SK_XF / 4);
    sk_cp_async_wait_all();
    if (gamma_staged) __syncthreads(); else __syncwarp();
    // whole rows of 1024 or 2048 columns in one piece, the norm's weights parked: straight-line code
    const bool fast8 = gamma_staged && k_cta == 0 && a.k_per_cta >= a.K && nv == 256;
    const bool fast16 = gamma_staged && k_cta == 0 && a.k_per_cta >= a.K && nv == 512;
    for (int r = warp; r < MP; r += SK_WARPS) {
      bf16* row = xs + (size_t)r * a.xs_stride;
      if (r < a.M && (fast8 || fast16)) {
        if (r != warp) { __syncwarp(); request_piece(a.xf + (size_t)r * a.lda, 0); sk_cp_async_wait_all(); __syncwarp(); }
        if (fast8) norm_row_fast<8>(piece, gamma_s, row, lane, a.K, a.eps);
        else norm_row_fast<16>(piece, gamma_s, row, lane, a.K, a.eps);
        for (int k = a.K + lane * 4; k < a.k_per_cta; k += 128) *(uint2*)(row + k) = make_uint2(0, 0);
        continue;
      }
      if (r >= a.M) {
        for (int k = lane * 4; k < a.k_per_cta; k += 128) *(uint2*)(row + k) = make_uint2(0, 0);
        continue;
      }
      const float* xrow = a.xf + (size_t)r * a.lda;
      float ss = 0.f;
      for (int pc = 0; pc < n_pieces; ++pc) {
        if (pc > 0 || r != warp) { __syncwarp(); request_piece(xrow, pc); sk_cp_async_wait_all(); __syncwarp(); }
        const int cnt = min(nv - pc * (SK_XF / 4), SK_XF / 4);
        for (int i = lane; i < cnt; i += 32) {
          float4 v = piece[i];
          ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
      }
      ss = warp_sum(ss);
      const float sc = 1.0f / sqrtf(ss / (float)a.K + a.eps);
      for (int pc = 0; pc < n_pieces; ++pc) {
        if (n_pieces > 1) { __syncwarp(); request_piece(xrow, pc); sk_cp_async_wait_all(); __syncwarp(); }
        const int v0 = pc * (SK_XF / 4), cnt = min(nv - v0, SK_XF / 4);
        for (int i = lane; i < cnt; i += 32) {
          int k = 4 * (v0 + i) - k_cta;
          if (k < 0 || k >= a.k_per_cta) continue;
          float4 x = piece[i], gw = gamma_staged ? gamma_s[v0 + i] : wr[v0 + i];
          __nv_bfloat162 p0 = __floats2bfloat162_rn((x.x * sc) * gw.x, (x.y * sc) * gw.y);
          __nv_bfloat162 p1 = __floats2bfloat162_rn((x.z * sc) * gw.z, (x.w * sc) * gw.w);
          uint2 val; val.x = *(unsigned*)&p0; val.y = *(unsigned*)&p1;
          *(uint2*)(row + k) = val;
        }
      }
      // columns of the slice past K (the last split of a K that the splits do not divide)
      for (int k = max(a.K - k_cta, 0) + lane * 4; k < a.k_per_cta; k += 128) *(uint2*)(row + k) = make_uint2(0, 0);
    }
  } else {
    sk_cp_async_wait_all();
  }
  __syncthreads();
  FELLM_TRACE_MARK(0);

  // ---- rounds of SK_U chunks; the round after next is requested before this one is multiplied
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
  float* slots = (float*)(smem + (size_t)MT * 8 * a.xs_stride * sizeof(bf16));      // [warp][tile of warp][16][MP], split-K only
  const bf16* xw = xs + (size_t)g * a.xs_stride + wk * a.k_per_warp + c * 8;
  const bool direct = a.splits == 1 && a.warps_k == 1;

  auto compute_round = [&](int tl, int rr, const uint4* w0, const uint4* w1) {
    const int n_valid = n_chunks - rr * SK_U;                        // warp-uniform
    const bf16* xr0 = xw + rr * (SK_U * KCHUNK);
#pragma unroll
    for (int u = 0; u < SK_U; ++u) {
      if (u < n_valid) {
        unsigned fa[4] = {w0[u].x, w1[u].x, w0[u].y, w1[u].y};
        unsigned fb[4] = {w0[u].z, w1[u].z, w0[u].w, w1[u].w};
        const bf16* xr = xr0 + u * KCHUNK;
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

  int ctl = 0, crr = 0;
  for (int r = 0; r < total_rounds; r += 2) {
    compute_round(ctl, crr, wA0, wA1); advance(ctl, crr);
    if (r + 2 < total_rounds) { load_round(ltl, lrr, wA0, wA1); advance(ltl, lrr); }
    if (r + 1 < total_rounds) {
      compute_round(ctl, crr, wB0, wB1); advance(ctl, crr);
      if (r + 3 < total_rounds) { load_round(ltl, lrr, wB0, wB1); advance(ltl, lrr); }
    }
  }
  FELLM_TRACE_MARK(1);
  if (direct) return;

  // ---- split K: sum the partial slabs over the cluster's ranks and the CTA's K warps, in that
  // order; every (rank, K warp) finishes a share of each slab's outputs
  if (a.splits > 1) cg::this_cluster().sync(); else __syncthreads();
  FELLM_TRACE_MARK(2);
  const int workers = a.splits << a.log2_warps_k, me = (split << a.log2_warps_k) + wk;
  const float* slab_slots = slots + (size_t)(wn << a.log2_warps_k) * a.tiles_per_warp * SK_ROWS * MP;   // K warp 0 of this slab
  const int warp_stride = a.tiles_per_warp * SK_ROWS * MP;
  for (int tl = 0; tl < my_tiles; ++tl) {
    int n0 = (first_tile + tl * tile_stride) * SK_ROWS;
    const float* mine = slab_slots + (size_t)tl * SK_ROWS * MP;
    const int units = (EPI == EPI_SWIGLU ? 8 : SK_ROWS) * a.M;          // outputs of the slab
    for (int i = me * 32 + lane; i < units; i += workers * 32) {
      int m, j;
      if (EPI == EPI_SWIGLU) { m = i >> 3; j = i & 7; } else { m = i >> 4; j = i & 15; }
      const int n = n0 + j;
      const bool live = n < a.N;
      const size_t o = (size_t)m * a.ldo + n;
      float old = 0.f;
      if (EPI == EPI_ACC && live) old = ((float*)a.out)[o];          // asked for before the partial sums
      const float* mine_e = mine + j * MP + m;
      // partial sums in the order (rank, K warp), requested RG at a time
      constexpr int RG = 8;
      float v0 = 0.f, v1 = 0.f;
      for (int q0 = 0; q0 < workers; q0 += RG) {
        float p0[RG], p1[RG];
#pragma unroll
        for (int q = 0; q < RG; ++q) {
          int idx = q0 + q;
          p0[q] = 0.f; p1[q] = 0.f;
          if (idx < workers) {
            int sr = idx >> a.log2_warps_k, w = idx & (a.warps_k - 1);
            const float* p = a.splits > 1 ? cg::this_cluster().map_shared_rank(mine_e, sr) : mine_e;
            p0[q] = p[w * warp_stride];
            if (EPI == EPI_SWIGLU) p1[q] = p[w * warp_stride + 8 * MP];
          }
        }
#pragma unroll
        for (int q = 0; q < RG; ++q) {
          if (q0 + q < workers) { v0 += p0[q]; if (EPI == EPI_SWIGLU) v1 += p1[q]; }
        }
      }
      if (!live) continue;
      if (EPI == EPI_SWIGLU) {
        if (a.bias) { v0 += a.bias[n]; v1 += a.bias[n + 8]; }
        ((bf16*)a.out)[(size_t)m * a.ldo + (n0 >> 1) + j] = __float2bfloat16_rn((v0 / (1.0f + expf(-v0))) * v1);
      } else {
        if (a.bias) v0 += a.bias[n];
        if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(v0);
        else if (EPI == EPI_ACC) ((float*)a.out)[o] = old + v0;
        else ((float*)a.out)[o] = v0;
      }
    }
  }
  if (a.splits > 1) cg::this_cluster().sync();           // nobody leaves while its slabs are being read
}

// ---------------------------------------------------------------- the single-shot kernel
// The decode step's products: M <= 64 rows, every (slab, K slice) has a warp of its own, a slice is
// at most LEAN_CH whole chunks, N is a multiple of 16, the CTA's K range of x fits shared memory.
// One pass, no loops over slabs or rounds:
// the same sums in the same order as gemm_skinny_kernel, in a third of the instructions (a warp's
// serial instruction stream is what a product of a few microseconds waits for).
#define LEAN_CH 10
#define LEAN_TPW 8

template <int OFF>
__device__ __forceinline__ uint4 ldg_stream_at(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "n"(OFF));
  return v;
}

template <int U, int N>
struct LeanLoad {
  static __device__ __forceinline__ void run(const bf16* p0, const bf16* p1, uint4* w0, uint4* w1, int n_chunks) {
    if (U < 8 || U < n_chunks) {                       // the first 8 chunks are there (n_chunks >= 8), the rest are tested
      w0[U] = ldg_stream_at<U * KCHUNK * 2>(p0);
      w1[U] = ldg_stream_at<U * KCHUNK * 2>(p1);
    }
    LeanLoad<U + 1, N>::run(p0, p1, w0, w1, n_chunks);
  }
};
template <int N>
struct LeanLoad<N, N> {
  static __device__ __forceinline__ void run(const bf16*, const bf16*, uint4*, uint4*, int) {}
};

template <int MT, int EPI, bool NORM, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 2 : 1) gemm_lean_kernel(SkinnyArgs a) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_SKINNY + 32 * (EPI == EPI_CONV ? EPI_STORE : (EPI == EPI_ARGMAX ? EPI_F32 : EPI)));
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int MP = MT * 8;
  __shared__ unsigned long long arg_best[EPI == EPI_ARGMAX ? MT * 8 : 1];     // the CTA's best key of each row
  if (EPI == EPI_ARGMAX && threadIdx.x < MT * 8) arg_best[threadIdx.x] = 0ull;  // seen by all behind the barrier before the sums
  __shared__ float rs_scale[MT * 8];                   // the rows' norm factors when x comes pre-weighted (a.rs_ssq)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = a.splits > 1 ? (int)cg::this_cluster().block_rank() : 0;
  const int wn = warp >> a.log2_warps_k, wk = warp & (a.warps_k - 1);
  const int k_cta = split * a.k_per_cta;
  const int n_chunks = a.chunks_per_warp;              // 8..LEAN_CH, the same for every warp
  // the warp's slabs: tile, tile + tile_stride, ...: tiles_per_warp of them (some past the last slab)
  const int tile = blockIdx.y * (WARPS >> a.log2_warps_k) + wn;
  const int tile_stride = gridDim.y * (WARPS >> a.log2_warps_k);
  const int tpw = a.tiles_per_warp;
  bf16* xs = (bf16*)smem;
  const int nv = a.K >> 2;
  float4* piece = (float4*)(smem + a.xf_offset) + (size_t)(warp < MP ? warp : 0) * nv;     // NORM: the float32 row of warp < MP
  const unsigned piece_s = (unsigned)__cvta_generic_to_shared(piece);

  auto request_row = [&](int r) {                      // NORM: float32 row r into the warp's piece
    const float* xrow = a.xf + (size_t)r * a.lda;
    for (int i = lane; i < nv; i += 32) sk_cp_async16(piece_s + 16u * i, xrow + 4 * i);
  };
  auto request_x = [&]() {
    if (NORM) {
      if (warp < a.M && warp < MP) request_row(warp);
    } else {
      const int vec_per_row = a.k_per_cta >> 3;
      const unsigned xs_s = (unsigned)__cvta_generic_to_shared(xs);
      for (int r = warp; r < MP; r += WARPS) {
        bf16* dst = xs + (size_t)r * a.xs_stride;
        if (r < a.M) {
          const bf16* src = a.x + (size_t)r * a.lda + k_cta;
          const unsigned dst_s = xs_s + 2u * (unsigned)(r * a.xs_stride);
          for (int vv = lane; vv < vec_per_row; vv += 32) sk_cp_async16(dst_s + 16u * vv, src + vv * 8);
        } else {
          for (int vv = lane; vv < vec_per_row; vv += 32) *(uint4*)(dst + vv * 8) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  };

  // ---- requests: the norm's weights and W never wait for the kernel before this one; x is asked
  // for first when the launch is an ordinary one (so that it does not queue behind W), after the
  // wait when the kernel runs as a programmatic dependent
  if (NORM) {
    const unsigned gs = (unsigned)__cvta_generic_to_shared(smem + a.gamma_offset);
    for (int i = threadIdx.x; i < nv; i += WARPS * 32) sk_cp_async16(gs + 16u * i, a.norm_w + 4 * i);
  }
  if (!a.pdl) request_x();
  uint4 w0[LEAN_CH], w1[LEAN_CH];
  const bf16* w_base = a.W + (size_t)g * a.ldw + k_cta + wk * a.k_per_warp + c * 8;
  if (tile < a.n_tiles) {
    const bf16* p0 = w_base + (size_t)tile * SK_ROWS * a.ldw;
    LeanLoad<0, LEAN_CH>::run(p0, p0 + (size_t)8 * a.ldw, w0, w1, n_chunks);
  }
  // EPI_ACC with a norm to hand on: the next norm's weight for the value this thread finishes first
  // which share of a slab's outputs this warp finishes: K warp w of rank r is number w * ranks + r of them, so that
  // the first shares of a slab go to different ranks (a slab of 8 tokens has four shares of 32 outputs)
  const int me = wk * a.splits + split;
  const int first_unit = me * 32 + lane;
  float next_w_first = 0.f;
  if (EPI == EPI_ACC && a.nn_x && first_unit < SK_ROWS * a.M && tile < a.n_tiles) next_w_first = a.nn_w[tile * SK_ROWS + (first_unit & 15)];
  if (threadIdx.x < 32)                                   // (a lane a piece: one thread's loop was 40 turns long for a wide matrix)
    l2_prefetch_share(a.next_w, a.next_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, gridDim.x * gridDim.y * gridDim.z, lane, 32);
  pdl_launch_dependents();
  if (a.pdl) {
    pdl_wait();
    request_x();
  }
  FELLM_TRACE_WAITED();
  // the rows' sums of squares come in parts (at most 128 a row): warp w asks for those of rows w and (with more rows
  // than warps) w + WARPS now, beside x; a lane adds its parts up once x is there (one register a row is then held
  // through the product: held as they came, eight of them cost the kernel its weights in flight), and the lanes'
  // sums are added behind the product, where nobody waits for them.  Always in the same order.
  constexpr int RS_H = (MT * 8 > WARPS) ? 2 : 1;
  float rs_part[RS_H][4], rs_sum[RS_H];
  if (a.rs_ssq) {
#pragma unroll
    for (int h = 0; h < RS_H; ++h) {
      const int r = warp + h * WARPS;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int p = lane + 32 * q;
        rs_part[h][q] = (r < a.M && p < a.rs_parts) ? a.rs_ssq[(size_t)r * a.rs_parts + p] : 0.f;
      }
    }
  }
  // EPI_ACC: the value this thread adds to first is asked for now too
  float old_first = 0.f;
  if (EPI == EPI_ACC && first_unit < SK_ROWS * a.M && tile < a.n_tiles)
    old_first = ((const float*)a.out)[(size_t)(first_unit >> 4) * a.ldo + tile * SK_ROWS + (first_unit & 15)];

  // EPI_CONV: thread (channel j of the CTA's 16, token m) asks for its taps and its state now; they
  // are used after the product
  float cv_hist[SK_MAX_LC - 1], cv_w[SK_MAX_LC], cv_bias = 0.f;
  float* cv_state = nullptr;
  const bool conv_thread = EPI == EPI_CONV && (int)threadIdx.x < SK_ROWS * a.M;
  if (EPI == EPI_CONV && conv_thread) {
    const int j = threadIdx.x & 15, m = threadIdx.x >> 4, ch = blockIdx.y * SK_ROWS + j, d = a.N / 3;
    cv_state = a.conv_state + (size_t)a.row_slot[m] * a.conv_slot_stride + ch;
#pragma unroll
    for (int t = 0; t < SK_MAX_LC - 1; ++t) cv_hist[t] = t < a.conv_taps - 1 ? cv_state[(size_t)t * d] : 0.f;
#pragma unroll
    for (int t = 0; t < SK_MAX_LC; ++t) cv_w[t] = t < a.conv_taps ? a.conv_w[(size_t)ch * a.conv_taps + t] : 0.f;
    if (a.conv_bias) cv_bias = a.conv_bias[ch];
  }

  sk_cp_async_wait_all();
  if (a.rs_ssq) {
#pragma unroll
    for (int h = 0; h < RS_H; ++h) rs_sum[h] = (rs_part[h][0] + rs_part[h][1]) + (rs_part[h][2] + rs_part[h][3]);
  }
  if (NORM) {
    // RMSNorm (crates/backend-cpu/src/kernels/norm.rs:6-39): a warp per row, whole rows
    const float4* gamma_s = (const float4*)(smem + a.gamma_offset);
    __syncthreads();
    for (int r = warp; r < MP; r += WARPS) {
      bf16* row = xs + (size_t)r * a.xs_stride;
      if (r < a.M) {
        if (r != warp) { __syncwarp(); request_row(r); sk_cp_async_wait_all(); __syncwarp(); }
        if (nv == 256) norm_row_fast<8>(piece, gamma_s, row, lane, a.K, a.eps);
        else if (nv == 512) norm_row_fast<16>(piece, gamma_s, row, lane, a.K, a.eps);
        else {
          float ss = 0.f;
          for (int i = lane; i < nv; i += 32) {
            const float4 v = piece[i];
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
          }
          ss = warp_sum(ss);
          const float sc = 1.0f / sqrtf(ss / (float)a.K + a.eps);
          for (int i = lane; i < nv; i += 32) {
            const float4 v = piece[i], gw = gamma_s[i];
            __nv_bfloat162 q0 = __floats2bfloat162_rn((v.x * sc) * gw.x, (v.y * sc) * gw.y);
            __nv_bfloat162 q1 = __floats2bfloat162_rn((v.z * sc) * gw.z, (v.w * sc) * gw.w);
            uint2 val; val.x = *(unsigned*)&q0; val.y = *(unsigned*)&q1;
            *(uint2*)(row + 4 * i) = val;
          }
        }
      } else {
        for (int k = lane * 4; k < a.K; k += 128) *(uint2*)(row + k) = make_uint2(0, 0);
      }
    }
  }
  __syncthreads();
  FELLM_TRACE_MARK(0);

  // ---- the warp's slice of each of its slabs, four token tiles (32 rows of x) at a time; the next
  // slab's weights are asked for as soon as this one's are used up
  constexpr int TP = MT > 4 ? 4 : MT;
  float* slots = (float*)(smem + (size_t)MP * a.xs_stride * sizeof(bf16));      // [warp][slab of warp][16][MP]
  const bf16* xw = xs + (size_t)g * a.xs_stride + wk * a.k_per_warp + c * 8;
  for (int tl = 0; tl < tpw; ++tl) {
    const int tile_l = tile + tl * tile_stride;
    if (tile_l >= a.n_tiles) break;
    float* p = slots + (size_t)(warp * tpw + tl) * SK_ROWS * MP;
#pragma unroll
    for (int pass = 0; pass < MT / TP; ++pass) {
      // up to 16 tokens: the two halves of a chunk add into sums of their own, so that an MMA waits for the one
      // two before it, not for the one before it (the sums are added at the end; more tokens have MMAs enough)
      constexpr int CH = TP <= 2 ? 2 : 1;
      float acc[TP][CH][4];
#pragma unroll
      for (int t = 0; t < TP; ++t)
#pragma unroll
        for (int h = 0; h < CH; ++h) { acc[t][h][0] = acc[t][h][1] = acc[t][h][2] = acc[t][h][3] = 0.f; }
#pragma unroll
      for (int u = 0; u < LEAN_CH; ++u) {
        if (u < 8 || u < n_chunks) {
          unsigned fa[4] = {w0[u].x, w1[u].x, w0[u].y, w1[u].y};
          unsigned fb[4] = {w0[u].z, w1[u].z, w0[u].w, w1[u].w};
#pragma unroll
          for (int t = 0; t < TP; ++t) {
            uint4 b = *(const uint4*)(xw + u * KCHUNK + (size_t)(pass * TP + t) * 8 * a.xs_stride);
            mma16816(acc[t][0], fa, b.x, b.y);
            mma16816(acc[t][CH - 1], fb, b.z, b.w);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < TP; ++t) {
        if (CH == 2) {
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[t][0][e] += acc[t][1][e];
        }
        *(float2*)(p + g * MP + (pass * TP + t) * 8 + 2 * c) = make_float2(acc[t][0][0], acc[t][0][1]);
        *(float2*)(p + (g + 8) * MP + (pass * TP + t) * 8 + 2 * c) = make_float2(acc[t][0][2], acc[t][0][3]);
      }
    }
    if (tl + 1 < tpw && tile_l + tile_stride < a.n_tiles) {
      const bf16* p0 = w_base + (size_t)(tile_l + tile_stride) * SK_ROWS * a.ldw;
      LeanLoad<0, LEAN_CH>::run(p0, p0 + (size_t)8 * a.ldw, w0, w1, n_chunks);
    }
  }
  if (a.rs_ssq) {
    // RMSNorm's factor of each row (crates/backend-cpu/src/kernels/norm.rs:6-39)
#pragma unroll
    for (int h = 0; h < RS_H; ++h) {
      const int r = warp + h * WARPS;
      if (r < a.M) {                                   // (whole warps)
        const float ss = warp_sum(rs_sum[h]);
        if (lane == 0) rs_scale[r] = 1.0f / sqrtf(ss / (float)a.K + a.rs_eps);
      }
    }
  }
  FELLM_TRACE_MARK(1);
  const int warp_stride = tpw * SK_ROWS * MP;
  // K over a cluster: every CTA first adds up its own K warps (into the slot of K warp 0 of each slab, all threads
  // sharing the elements), so that what is read from the other ranks afterwards is one value a rank, not one a warp
  const bool own_first = a.splits > 1 && a.warps_k > 1;
  if (own_first) {
    __syncthreads();
    const int slab_elems = SK_ROWS * MP, slabs = (WARPS >> a.log2_warps_k) * tpw;
    for (int e = threadIdx.x; e < slabs * slab_elems; e += WARPS * 32) {
      const int sl = e / slab_elems, off = e - sl * slab_elems, wn_ = sl / tpw, tl_ = sl - wn_ * tpw;
      float* first = slots + (size_t)((wn_ << a.log2_warps_k) * tpw + tl_) * slab_elems + off;
      float v = first[0];
      for (int w = 1; w < a.warps_k; ++w) v += first[(size_t)w * warp_stride];
      first[0] = v;
    }
  }
  if (a.splits > 1) cg::this_cluster().sync(); else __syncthreads();
  FELLM_TRACE_MARK(2);

  // ---- sum the partial slabs over the cluster's ranks and the CTA's K warps, in that order; every
  // (rank, K warp) finishes a share of each slab's outputs
  const int workers = a.splits << a.log2_warps_k;
  for (int tl = 0; tl < tpw; ++tl) {
    const int tile_l = tile + tl * tile_stride;
    if (tile_l >= a.n_tiles) break;
    const int n0 = tile_l * SK_ROWS;
    const float* mine = slots + (size_t)((wn << a.log2_warps_k) * tpw + tl) * SK_ROWS * MP;      // K warp 0 of this slab
    const int units = (EPI == EPI_SWIGLU ? 8 : SK_ROWS) * a.M;
    for (int i0 = me * 32; i0 < units; i0 += workers * 32) {
      // (the warp stays whole for the shuffles of EPI_ARGMAX and EPI_ACC; units is a multiple of 16, so half
      // warps are in or out together)
      const bool live = i0 + lane < units;
      if (EPI != EPI_ARGMAX && EPI != EPI_ACC && !live) continue;
      const int i = live ? i0 + lane : 0;
      int m, j;
      if (EPI == EPI_SWIGLU) { m = i >> 3; j = i & 7; } else { m = i >> 4; j = i & 15; }
      const int n = n0 + j;
      const size_t o = (size_t)m * a.ldo + n;
      float old = 0.f, next_w = 0.f;
      if (EPI == EPI_ACC && live) {
        if (tl == 0 && i0 == me * 32) { old = old_first; next_w = next_w_first; }      // asked for long ago
        else {                                                       // asked for before the partial sums
          old = ((float*)a.out)[o];
          if (a.nn_x) next_w = a.nn_w[n];
        }
      }
      const float* mine_e = mine + j * MP + m;
      constexpr int RG = 8;
      float v0 = 0.f, v1 = 0.f;
      if (a.splits == 1) {
        // the CTA's own K warps, four at a time (their number is a power of two)
        for (int w0 = 0; w0 < a.warps_k; w0 += 4) {
          float p0[4], p1[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const bool on = w0 + q < a.warps_k;
            p0[q] = on ? mine_e[(w0 + q) * warp_stride] : 0.f;
            p1[q] = (EPI == EPI_SWIGLU && on) ? mine_e[(w0 + q) * warp_stride + 8 * MP] : 0.f;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (w0 + q < a.warps_k) { v0 += p0[q]; if (EPI == EPI_SWIGLU) v1 += p1[q]; }
          }
        }
      } else {
        const int parts = own_first ? a.splits : workers;             // a value a rank, or a value a (rank, K warp)
        for (int q0 = 0; q0 < parts; q0 += RG) {
          float p0[RG], p1[RG];
#pragma unroll
          for (int q = 0; q < RG; ++q) {
            const int idx = q0 + q;
            p0[q] = 0.f; p1[q] = 0.f;
            if (idx < parts) {
              const int sr = own_first ? idx : idx >> a.log2_warps_k, w = own_first ? 0 : idx & (a.warps_k - 1);
              const float* pp = a.splits > 1 ? cg::this_cluster().map_shared_rank(mine_e, sr) : mine_e;
              p0[q] = pp[w * warp_stride];
              if (EPI == EPI_SWIGLU) p1[q] = pp[w * warp_stride + 8 * MP];
            }
          }
#pragma unroll
          for (int q = 0; q < RG; ++q) {
            if (q0 + q < parts) { v0 += p0[q]; if (EPI == EPI_SWIGLU) v1 += p1[q]; }
          }
        }
      }
      if (a.rs_ssq) { const float sc = rs_scale[m]; v0 *= sc; if (EPI == EPI_SWIGLU) v1 *= sc; }
      if (EPI == EPI_SWIGLU) {
        if (a.bias) { v0 += a.bias[n]; v1 += a.bias[n + 8]; }
        ((bf16*)a.out)[(size_t)m * a.ldo + (n0 >> 1) + j] = __float2bfloat16_rn((v0 / (1.0f + expf(-v0))) * v1);
      } else if (EPI == EPI_CONV) {
        // B, C or X of (channel j, token m), rounded as the stored product would be
        if (a.bias) v0 += a.bias[n];
        ((float*)(smem + a.red_offset))[(wn * SK_ROWS + j) * MP + m] = __bfloat162float(__float2bfloat16_rn(v0));
      } else if (EPI == EPI_ARGMAX) {
        // the slab's 16 outputs of row m lie in one half warp: its best key, then one atomic a half warp
        if (a.bias) v0 += a.bias[n];
        unsigned long long key = live ? argmax_key(v0, n) : 0ull;
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o2);
          key = other > key ? other : key;
        }
        if (live && (lane & 15) == 0) atomicMax(&arg_best[m], key);
      } else {
        if (a.bias) v0 += a.bias[n];
        if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(v0);
        else if (EPI == EPI_ACC) {
          const float v = old + v0;
          if (live) ((float*)a.out)[o] = v;
          if (a.nn_x) {
            // the slab's 16 new values of row m lie in one half warp: their squares' sum is one part of the
            // row's; the value goes on weighted, the row's factor follows in the next product
            float sq = live ? v * v : 0.f;
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o2);
            if (live) {
              a.nn_x[(size_t)m * a.nn_ldx + n] = __float2bfloat16_rn(v * next_w);
              if ((lane & 15) == 0) a.nn_ssq[(size_t)m * a.n_tiles + tile_l] = sq;
            }
          }
        } else ((float*)a.out)[o] = v0;
      }
    }
  }
  if (EPI == EPI_ARGMAX) {
    __syncthreads();
    const int cta = blockIdx.y * gridDim.x + blockIdx.x, n_ctas = gridDim.x * gridDim.y;
    if (threadIdx.x < a.M) a.arg_keys[(size_t)threadIdx.x * n_ctas + cta] = arg_best[threadIdx.x];
  }
  if (EPI == EPI_CONV) {
    // the CTA's three slabs are B, C and X of its 16 channels (the weight rows come in blocks of
    // 16 B / 16 C / 16 X rows): bx = B*X; conv = bx*w[Lc-1] + sum_t state[t]*w[t]; y = C*(conv + bias);
    // the state moves on by one (crates/backend-cpu/src/kernels/shortconv.rs:61-106).  Nobody else
    // reads or writes these channels' state.
    __syncthreads();
    if (conv_thread) {
      const int j = threadIdx.x & 15, m = threadIdx.x >> 4, d = a.N / 3, H = a.conv_taps - 1;
      const float* red = (const float*)(smem + a.red_offset);
      const float bx = red[j * MP + m] * red[(2 * SK_ROWS + j) * MP + m];
      float wlast = 0.f;
#pragma unroll
      for (int t = 0; t < SK_MAX_LC; ++t) if (t == H) wlast = cv_w[t];
      float conv = bx * wlast;
#pragma unroll
      for (int t = 0; t < SK_MAX_LC - 1; ++t) if (t < H) conv = fmaf(cv_hist[t], cv_w[t], conv);
      ((bf16*)a.out)[(size_t)m * a.ldo + blockIdx.y * SK_ROWS + j] = __float2bfloat16_rn(red[(SK_ROWS + j) * MP + m] * (conv + cv_bias));
#pragma unroll
      for (int t = 0; t < SK_MAX_LC - 1; ++t) {
        if (t < H) cv_state[(size_t)t * d] = (t + 1 < H) ? cv_hist[t + 1 < SK_MAX_LC - 1 ? t + 1 : t] : bx;
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

// Which products are launched as programmatic dependents (launch class 1) by epilogue kind: all but
// the one with the convolution behind it.  A chain in which EVERY kernel starts early piles kernels
// up on the SMs ahead of the one that has to finish first: measured on B200 at batch 8 (16 layers of
// width 1024, one decode step replayed from a graph), 424 us with the convolution product in the
// chain, 399 us with it launched the ordinary way, 414 us with the convolution as a kernel of its
// own.  FELLM_B200_PDL_EPIS overrides the mask (bit = epilogue kind) for experiments.
static int pdl_class_of(int epi) {
  static int mask = -1;
  if (mask < 0) { const char* e = getenv("FELLM_B200_PDL_EPIS"); mask = e ? atoi(e) : 47; }
  return ((mask >> epi) & 1) ? 1 : 0;
}

template <int MT, int EPI>
static int launch(SkinnyArgs a, int ctas_y, cudaStream_t stream) {
  size_t smem = smem_bytes(MT, a.k_per_cta, a.splits == 1 && a.warps_k == 1, a.tiles_per_warp);
  a.gamma_offset = (int)smem;                              // the norm's weights, behind x and the partial slabs
  if (a.xf && a.K <= SK_GAMMA_MAX) smem += (size_t)a.K * sizeof(float);
  a.xf_offset = (int)smem;                                 // a float32 row piece per warp
  if (a.xf) smem += (size_t)SK_WARPS * (a.K < SK_XF ? a.K : SK_XF) * sizeof(float);
  auto kern = gemm_skinny_kernel<MT, EPI>;
  if (smem + 1024 > 48 * 1024) {                            // (the kernel's static shared memory counts toward the 48 KB too)
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int cls = pdl_class_of(EPI);
  a.pdl = pdl_enabled(cls) ? 1 : 0;
  return launch_k_class(cls, kern, dim3(a.splits, ctas_y, 1), dim3(SK_THREADS, 1, 1), smem, stream, a.splits, a);
}

template <int MT, int EPI, bool NORM, int WARPS>
static int launch_lean(SkinnyArgs a, int ctas_y, cudaStream_t stream) {
  size_t smem = (size_t)MT * 8 * x_stride(a.k_per_cta) * sizeof(bf16) + (size_t)WARPS * a.tiles_per_warp * SK_ROWS * MT * 8 * sizeof(float);
  a.gamma_offset = (int)smem;
  if (NORM) smem += (size_t)a.K * sizeof(float);
  a.xf_offset = (int)smem;
  if (NORM) smem += (size_t)(WARPS < MT * 8 ? WARPS : MT * 8) * a.K * sizeof(float);
  if (!NORM && MT <= 2 && a.xf) return FELLM_ERR_ARG;
  a.red_offset = (int)smem;
  if (EPI == EPI_CONV) smem += (size_t)3 * SK_ROWS * MT * 8 * sizeof(float);
  auto kern = gemm_lean_kernel<MT, EPI, NORM, WARPS>;
  if (smem + 1024 > 48 * 1024) {                            // (the kernel's static shared memory counts toward the 48 KB too)
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int cls = pdl_class_of(EPI);
  a.pdl = pdl_enabled(cls) ? 1 : 0;
  return launch_k_class(cls, kern, dim3(a.splits, ctas_y, 1), dim3(WARPS * 32, 1, 1), smem, stream, a.splits, a);
}

static size_t lean_smem(int mt, int warps, int k_per_cta, bool norm, int K, int tpw = 1) {
  size_t smem = (size_t)mt * 8 * x_stride(k_per_cta) * sizeof(bf16) + (size_t)warps * tpw * SK_ROWS * mt * 8 * sizeof(float);
  if (norm) smem += (size_t)K * sizeof(float) + (size_t)(warps < mt * 8 ? warps : mt * 8) * K * sizeof(float);
  return smem;
}

template <int EPI, int WARPS>
static int dispatch_lean_mt(const SkinnyArgs& a, int ctas_y, cudaStream_t s) {
  if (a.M <= 8) return a.xf ? launch_lean<1, EPI, true, WARPS>(a, ctas_y, s) : launch_lean<1, EPI, false, WARPS>(a, ctas_y, s);
  if (a.M <= 16) return a.xf ? launch_lean<2, EPI, true, WARPS>(a, ctas_y, s) : launch_lean<2, EPI, false, WARPS>(a, ctas_y, s);
  if (a.xf) return FELLM_ERR_SIZE;                       // the norm is fused for up to 16 rows
  if (a.M <= 32) return launch_lean<4, EPI, false, WARPS>(a, ctas_y, s);
  return launch_lean<8, EPI, false, WARPS>(a, ctas_y, s);
}

template <int EPI>
static int dispatch_lean(const SkinnyArgs& a, int ctas_y, int warps, cudaStream_t s) {
  return warps == 16 ? dispatch_lean_mt<EPI, 16>(a, ctas_y, s) : dispatch_lean_mt<EPI, 8>(a, ctas_y, s);
}

// The single-shot kernel's shape for a product, if it takes it: a (slab, K slice) per warp, whole
// chunks, whole slabs, whole-row norm.  CTAs of 8 warps (two to an SM where shared memory allows)
// or of 16 warps (one to an SM); K slices go to the warps of a CTA as far as the CTA's part of x
// fits shared memory, the rest over a cluster.  Among the shapes that run in one wave: fewest
// cluster ranks, then most CTAs.
struct LeanPlan { int warps, warps_k, splits, ctas_y, k_per_warp, tiles_per_warp; };
static bool plan_lean(int M, int N, int K, bool norm, LeanPlan* out) {
  if (M > 64 || (norm && M > 16) || N % SK_ROWS) return false;
  const int n_sm = fellm_sm_count();
  const int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8)), n_tiles = N / SK_ROWS;
  bool found = false;
  LeanPlan best = {};
  long long best_key = 0;
  // K slices of 8..LEAN_CH whole chunks: any number of them that is (a power of two of warps) x (up to 8 ranks of
  // a cluster), e.g. 1536 = 6 x 256 (2 warps x 3 ranks), 7168 = 28 x 256 (4 x 7), 3072 = 12 x 256 (4 x 3)
  for (int slices = 2; slices <= 128; ++slices) {
  if (K % slices || (K / slices) % KCHUNK) continue;
  const int kpw = K / slices;
  if (kpw < 8 * KCHUNK || kpw > LEAN_CH * KCHUNK) continue;
  for (int warps = 8; warps <= 16; warps *= 2) {
    int wk = 1;
    while (wk * 2 <= warps && slices % (wk * 2) == 0) wk *= 2;
    while (wk > 1 && lean_smem(mt, warps, kpw * wk, norm, K) > 200 * 1024) wk /= 2;
    const int sp = slices / wk, warps_n = warps / wk;
    if (sp > 8 || (norm && (sp > 1 || K > 4096))) continue;
    // slabs a warp walks over: as few as let the CTAs run in one wave (a wide product of a larger
    // model: up to LEAN_TPW, each slab's weights requested when the one before is used up)
    for (int tpw = 1; tpw <= LEAN_TPW; ++tpw) {
      const size_t smem = lean_smem(mt, warps, kpw * wk, norm, K, tpw);
      if (smem > 200 * 1024) break;
      const int ct = ceil_div(n_tiles, warps_n * tpw);
      const int per_sm = (warps == 8 && smem <= 100 * 1024) ? 2 : 1;
      if (ct * sp > n_sm * per_sm) continue;
      // order: fewest cluster ranks; fewest slabs a warp; not two CTAs to an SM where one would do
      // (x staged twice); then most CTAs
      const int crowded = (per_sm == 2 && ct * sp > n_sm) ? 1 : 0;
      const long long key = ((long long)sp << 48) | ((long long)tpw << 40) | ((long long)crowded << 32) | (long long)(100000 - ct * sp);
      if (!found || key < best_key) { best = LeanPlan{warps, wk, sp, ct, kpw, tpw}; best_key = key; found = true; }
      break;
    }
  }
  }
  if (found) *out = best;
  return found;
}

// Whether fellm_gemm_skinny would run this product on its single-shot kernel (1) or not (0).
FELLM_API int fellm_gemm_skinny_single_shot(int M, int N, int K, int norm) {
  LeanPlan p;
  return plan_lean(M, N, K, norm != 0, &p) ? 1 : 0;
}

// The norm handed on between two products (SkinnyArgs: nn_* and rs_*), announced for the module's next call.
// nn_w float32 [N], nn_x bfloat16 [M, ldx], nn_ssq float32 [M, N / 16]: the next call is an accumulate
// (epi 1) product of up to 16 rows that the single-shot kernel takes (fellm_gemm_skinny_single_shot).
FELLM_API int fellm_gemm_skinny_next_norm(const float* nn_w, void* nn_x, int nn_ldx, float* nn_ssq) {
  g_handoff.nn_w = nn_w; g_handoff.nn_x = nn_x; g_handoff.nn_ldx = nn_ldx; g_handoff.nn_ssq = nn_ssq;
  return 0;
}
// ssq float32 [M, parts]: the next call's x is a pre-weighted input; its sums are multiplied by the rows'
// factors 1 / sqrt(sum(ssq[m, :]) / K + eps).  Any epilogue, a product the single-shot kernel takes without norm.
FELLM_API int fellm_gemm_skinny_row_scale(const float* ssq, int parts, float eps) {
  g_handoff.rs_ssq = ssq; g_handoff.rs_parts = parts; g_handoff.rs_eps = eps;
  return 0;
}
static int apply_handoff(SkinnyArgs& a, const NormHandoff& h, int M, int N, int K, int epi) {
  if (!h.nn_x && !h.rs_ssq) return 0;
  LeanPlan p;
  if (M > 16 || (epi != EPI_CONV && !plan_lean(M, N, K, false, &p))) return FELLM_ERR_SIZE;
  if (h.nn_x && epi != EPI_ACC) return FELLM_ERR_ARG;
  if (h.nn_x && (!h.nn_w || !h.nn_ssq || h.nn_ldx < N)) return FELLM_ERR_ARG;
  if (h.rs_ssq && (h.rs_parts < 1 || h.rs_parts > 128)) return FELLM_ERR_ARG;
  a.nn_w = h.nn_w; a.nn_x = (bf16*)h.nn_x; a.nn_ssq = h.nn_ssq; a.nn_ldx = h.nn_ldx;
  a.rs_ssq = h.rs_ssq; a.rs_parts = h.rs_parts; a.rs_eps = h.rs_eps;
  return 0;
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
  const NormHandoff handoff = take_handoff();     // cleared whatever this call returns
  if (M <= 0 || N <= 0) return 0;
  if ((!x && !xf) || !W || !out || K <= 0) return FELLM_ERR_ARG;
  if (xf && !norm_w) return FELLM_ERR_ARG;
  if (M > 64 || (K % 8) || (ldw % 8)) return FELLM_ERR_SIZE;
  if (x && (lda % 8)) return FELLM_ERR_SIZE;
  if (xf && (lda % 4)) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && (N % 16)) return FELLM_ERR_SIZE;
  int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  const size_t smem_cap = 100 * 1024;                     // two CTAs per SM
  const int n_sm = fellm_sm_count();
  const int resident_warps = n_sm * 2 * SK_WARPS;
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
  bool plan_a = (long long)n_tiles * slices <= (long long)resident_warps * 6;      // up to six slabs a warp, still cut over K
  int ctas_y = 1, tiles_per_warp = 1, k_per_cta = 0;
  static int cps = 0;
  if (!cps) { const char* e = getenv("FELLM_B200_SKINNY_CPS"); cps = (e && e[0] == '1') ? 1 : 2; }
  if (plan_a) {
    k_per_cta = round_k(ceil_div(K, slices)) * warps_k;
    ctas_y = ceil_div(n_tiles, SK_WARPS / warps_k);
    if (ctas_y > (n_sm * cps) / splits) ctas_y = (n_sm * cps) / splits;
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
        if (ctas_y > (n_sm * 2) / splits) ctas_y = (n_sm * 2) / splits;
        if (ctas_y < 1) ctas_y = 1;
        tiles_per_warp = ceil_div(n_tiles, ctas_y * SK_WARPS);
        if (smem_bytes(mt, k_per_cta, splits == 1, tiles_per_warp) <= cap) { found = true; break; }
      }
    }
    if (!found) splits = 16;
    if (splits > 8) return FELLM_ERR_SIZE;
  }
  SkinnyArgs a = {};
  if (int bad = apply_handoff(a, handoff, M, N, K, epi)) return bad;
  { const NextWeights nw = take_next_weights(); a.next_w = nw.ptr; a.next_bytes = nw.bytes; }
  a.x = (const bf16*)x; a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.bias = bias; a.out = out;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldw = ldw; a.ldo = ldo; a.splits = splits;
  a.warps_k = warps_k; a.k_per_cta = k_per_cta; a.xs_stride = x_stride(k_per_cta);
  a.n_tiles = n_tiles; a.tiles_per_warp = tiles_per_warp;
  a.log2_warps_k = 0;
  while ((1 << a.log2_warps_k) < warps_k) ++a.log2_warps_k;
  a.k_per_warp = k_per_cta / warps_k;
  a.pdl = pdl_enabled(1) ? 1 : 0;
  LeanPlan lp;
  if (plan_lean(M, N, K, xf != nullptr, &lp)) {
    a.splits = lp.splits; a.warps_k = lp.warps_k; a.k_per_warp = lp.k_per_warp; a.k_per_cta = lp.k_per_warp * lp.warps_k;
    a.xs_stride = x_stride(a.k_per_cta); a.tiles_per_warp = lp.tiles_per_warp;
    a.log2_warps_k = 0;
    while ((1 << a.log2_warps_k) < lp.warps_k) ++a.log2_warps_k;
    a.chunks_per_warp = a.k_per_warp / KCHUNK;
    switch (epi) {
      case EPI_STORE: return dispatch_lean<EPI_STORE>(a, lp.ctas_y, lp.warps, stream);
      case EPI_ACC: return dispatch_lean<EPI_ACC>(a, lp.ctas_y, lp.warps, stream);
      case EPI_SWIGLU: return dispatch_lean<EPI_SWIGLU>(a, lp.ctas_y, lp.warps, stream);
      case EPI_F32: return dispatch_lean<EPI_F32>(a, lp.ctas_y, lp.warps, stream);
      default: return FELLM_ERR_ARG;
    }
  }
  if (a.nn_x || a.rs_ssq) return FELLM_ERR_SIZE;           // only the single-shot kernel hands a norm on
  switch (epi) {
    case EPI_STORE: return dispatch_mt<EPI_STORE>(a, ctas_y, stream);
    case EPI_ACC: return dispatch_mt<EPI_ACC>(a, ctas_y, stream);
    case EPI_SWIGLU: return dispatch_mt<EPI_SWIGLU>(a, ctas_y, stream);
    case EPI_F32: return dispatch_mt<EPI_F32>(a, ctas_y, stream);
    default: return FELLM_ERR_ARG;
  }
}

// Greedy tokens without the logits: argmax_n of x W^T (+ bias) for every row of a decode step of up to 16
// rows (FeLLM: bf16_matmul_rows then argmax_token, plugins/cuda_kernels/src/oxide_kernels.rs:3165,116).
// The single-shot product's CTAs each leave the best (value, index) of their part of a row as a key; a
// second, tiny kernel takes the best key of each row.  Ties go to the lower index.
__global__ void __launch_bounds__(32) argmax_keys_kernel(const unsigned long long* __restrict__ keys, int n_ctas, int* __restrict__ out_tokens) {
  FELLM_TRACE_SCOPE(TRACE_ARGMAX_FINAL);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  const int row = blockIdx.x, lane = threadIdx.x;
  unsigned long long best = 0ull;
  for (int c = lane; c < n_ctas; c += 32) { const unsigned long long k = keys[(size_t)row * n_ctas + c]; best = k > best ? k : best; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { const unsigned long long k = __shfl_xor_sync(0xffffffffu, best, o); best = k > best ? k : best; }
  if (lane == 0) out_tokens[row] = best ? (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull)) : 0;
}

// Keys (8 bytes each) fellm_gemm_skinny_argmax needs for this product, or 0 if it does not take it.
FELLM_API long long fellm_gemm_skinny_argmax_scratch(int M, int N, int K, int norm) {
  LeanPlan lp;
  if (M < 1 || M > 16 || (K % 8) || !plan_lean(M, N, K, norm != 0, &lp)) return 0;
  return (long long)M * lp.splits * lp.ctas_y;
}

// x / xf / norm_w / eps as fellm_gemm_skinny; keys: fellm_gemm_skinny_argmax_scratch(...) entries;
// out_tokens: int32 [M].  FELLM_ERR_SIZE where the single-shot product does not take the sizes.
FELLM_API int fellm_gemm_skinny_argmax(const void* x, const float* xf, const float* norm_w, float eps, const void* W,
                                       const float* bias, unsigned long long* keys, int* out_tokens, int M, int N, int K,
                                       int lda, int ldw, cudaStream_t stream) {
  const NormHandoff handoff = take_handoff();     // cleared whatever this call returns
  if (M <= 0 || N <= 0) return 0;
  if ((!x && !xf) || !W || !keys || !out_tokens || K <= 0 || (xf && !norm_w)) return FELLM_ERR_ARG;
  if (M > 16 || (K % 8) || (ldw % 8) || (x && (lda % 8)) || (xf && (lda % 4))) return FELLM_ERR_SIZE;
  LeanPlan lp;
  if (!plan_lean(M, N, K, xf != nullptr, &lp)) return FELLM_ERR_SIZE;
  SkinnyArgs a = {};
  if (int bad = apply_handoff(a, handoff, M, N, K, EPI_ARGMAX)) return bad;
  { const NextWeights nw = take_next_weights(); a.next_w = nw.ptr; a.next_bytes = nw.bytes; }
  a.x = (const bf16*)x; a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.bias = bias; a.out = nullptr;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldw = ldw; a.ldo = 0;
  a.n_tiles = N / SK_ROWS;
  a.splits = lp.splits; a.warps_k = lp.warps_k; a.log2_warps_k = 0;
  while ((1 << a.log2_warps_k) < lp.warps_k) ++a.log2_warps_k;
  a.k_per_warp = lp.k_per_warp; a.k_per_cta = lp.k_per_warp * lp.warps_k; a.xs_stride = x_stride(a.k_per_cta);
  a.tiles_per_warp = lp.tiles_per_warp;
  a.chunks_per_warp = a.k_per_warp / KCHUNK;
  a.arg_keys = keys;
  int e = dispatch_lean<EPI_ARGMAX>(a, lp.ctas_y, lp.warps, stream);
  if (e) return e;
  return launch_k(argmax_keys_kernel, dim3(M), dim3(32), 0, stream, 1, (const unsigned long long*)keys, lp.splits * lp.ctas_y, out_tokens);
}

// The input product of a ShortConv mixer with the gated convolution behind it, for a decode step:
// every row is one token of its own request.  W [3d, K]: rows in blocks of 16 channels, 16 B rows,
// 16 C rows, 16 X rows (bias, if any, in the same order); y [M, d] = C * conv(B*X) in bfloat16;
// state: this layer's slots, [Lc-1, d] float32 each, slot_stride floats apart, advanced by one
// token; row_slot [M].  Takes M <= 16, K in 1024..1280 with K % 128 == 0 (four K slices of whole
// chunks), d % 16 == 0, d <= 16 * the SM count; FELLM_ERR_SIZE otherwise (fellm_gemm_skinny_conv_takes asks).
static bool conv_shape_ok(int M, int N, int K, int taps) {
  return M >= 1 && M <= 16 && N % 48 == 0 && N / 48 <= fellm_sm_count() && K % (4 * KCHUNK) == 0 && K / 4 >= 8 * KCHUNK &&
         K / 4 <= LEAN_CH * KCHUNK && taps >= 2 && taps <= SK_MAX_LC;
}
FELLM_API int fellm_gemm_skinny_conv_takes(int M, int N, int K, int taps) { return conv_shape_ok(M, N, K, taps) ? 1 : 0; }

FELLM_API int fellm_gemm_skinny_conv(const void* x, const float* xf, const float* norm_w, float eps, const void* W,
                                     const float* bias, const float* conv_w, const float* conv_bias, float* state,
                                     long long slot_stride, const int* row_slot, int taps, void* y, int M, int N, int K,
                                     int lda, int ldw, int ldo, cudaStream_t stream) {
  const NormHandoff handoff = take_handoff();     // cleared whatever this call returns
  if (M <= 0) return 0;
  if ((!x && !xf) || !W || !y || !conv_w || !state || !row_slot || (xf && !norm_w)) return FELLM_ERR_ARG;
  if (!conv_shape_ok(M, N, K, taps) || (ldw % 8) || (x && (lda % 8)) || (xf && (lda % 4)) || (xf && K > 4096)) return FELLM_ERR_SIZE;
  SkinnyArgs a = {};
  if (int bad = apply_handoff(a, handoff, M, N, K, EPI_CONV)) return bad;
  { const NextWeights nw = take_next_weights(); a.next_w = nw.ptr; a.next_bytes = nw.bytes; }
  a.x = (const bf16*)x; a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.bias = bias; a.out = y;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldw = ldw; a.ldo = ldo;
  a.splits = 1; a.warps_k = 4; a.log2_warps_k = 2; a.k_per_warp = K / 4; a.k_per_cta = K; a.xs_stride = x_stride(K);
  a.n_tiles = N / SK_ROWS; a.tiles_per_warp = 1; a.chunks_per_warp = a.k_per_warp / KCHUNK; a.pdl = pdl_enabled(1) ? 1 : 0;
  a.conv_w = conv_w; a.conv_bias = conv_bias; a.conv_state = state; a.row_slot = row_slot; a.conv_slot_stride = slot_stride;
  a.conv_taps = taps;
  const int ctas = N / 48;
  if (M <= 8) return xf ? launch_lean<1, EPI_CONV, true, 12>(a, ctas, stream) : launch_lean<1, EPI_CONV, false, 12>(a, ctas, stream);
  return xf ? launch_lean<2, EPI_CONV, true, 12>(a, ctas, stream) : launch_lean<2, EPI_CONV, false, 12>(a, ctas, stream);
}

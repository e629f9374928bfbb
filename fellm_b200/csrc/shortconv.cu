// Gated short causal depthwise convolution over portions of prompts and single decoded tokens,
// with the per-request rolling state kept on the device.
//
// FeLLM counterpart: shortconv_mix / shortconv_mix_rows, one token per request
// (plugins/cuda_kernels/src/oxide_kernels.rs:3054-3096,3527-3572;
// crates/backend-cpu/src/kernels/shortconv.rs:61-106):
//   bx = B*X;  conv_c = bx_c*w[c,Lc-1] + sum_{t<Lc-1} state[t,c]*w[c,t];  y = C*conv;
//   state <- shift left, append bx.
// Here a request may bring any number of tokens in a step.  Token j of a portion reads bx of
// tokens j-(Lc-1)..j-1: from the portion itself where they lie in it, from the state slot
// otherwise.  The taps are summed in the order above for every token, so the float32 result
// is bit-equal however a prompt is cut.
//
// One reader and one writer per state element: the first Lc-1 tokens of each item (the only ones
// that read the state) and the state update are done by the same thread ("head" blocks); all
// other rows are independent ("body" blocks).
#include "common.cuh"

#define MAX_LC 8
#define BODY_ROWS 8

// Column of (part p = 0 B / 1 C / 2 X, channel c) in a row of the input product's output: thirds
// [B | C | X], or, `blocked`, blocks of 16 channels [B16 | C16 | X16] (the weight rows are then
// ordered so that one CTA of the decode product holds B, C and X of its channels).
__device__ __forceinline__ int sc_col(int p, int c, int d, int blocked) {
  return blocked ? (c >> 4) * 48 + p * 16 + (c & 15) : p * d + c;
}

__device__ __forceinline__ void sc_unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// Body rows, bfloat16, d % 8 == 0: a thread takes 8 consecutive channels (16-byte loads) of
// BODY_ROWS consecutive rows.  Its taps stay in registers and so do the products B*X of the Lc-1
// rows before the one it is at, so that a row costs three loads (B, X, C) and is read once, plus
// the Lc-1 rows before the tile.  Rows are asked for four at a time, before it is known whether
// they are body rows (row -> item -> item start are two dependent loads): rows before the batch's
// first are clamped, and a head row's result is dropped.  Same sums, in the same order, as the
// scalar path.  LC = taps (2..5; other counts take the scalar path).
template <int LC>
__device__ void shortconv_body_vec(const bf16* __restrict__ bcx, const float* __restrict__ w,
                                   const float* __restrict__ conv_bias, const int* __restrict__ item_start,
                                   const int* __restrict__ row_item, bf16* __restrict__ y, int T, int d, int blocked) {
  constexpr int H = LC - 1, RB = 4;
  // the threads of a grid row (all blocks along x) are laid over [tiles][groups of 8 channels]
  const int groups = d / 8, lin = blockIdx.x * blockDim.x + threadIdx.x;
  const int tiles_per_y = (gridDim.x * blockDim.x) / groups;      // >= 8: a grid row has a thread per channel
  const int tile_in_y = lin / groups;
  if (tile_in_y >= tiles_per_y) return;
  const int c0 = (lin - tile_in_y * groups) * 8;
  const int r0 = (blockIdx.y * tiles_per_y + tile_in_y) * BODY_ROWS;
  if (r0 >= T) return;
  const size_t ld = (size_t)3 * d;
  const int cb = sc_col(0, c0, d, blocked), cc = sc_col(1, c0, d, blocked), cx = sc_col(2, c0, d, blocked);   // 8 channels stay in one block
  float wt[LC][8], bias[8], win[H > 0 ? H : 1][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
#pragma unroll
    for (int t = 0; t < LC; ++t) wt[t][e] = w[(size_t)(c0 + e) * LC + t];
    bias[e] = conv_bias ? conv_bias[c0 + e] : 0.f;
  }
#pragma unroll
  for (int t = 0; t < H; ++t) {                              // B*X of the rows before the tile, oldest first
    const int rp = r0 - H + t;
    const bf16* pr = bcx + (size_t)(rp < 0 ? 0 : rp) * ld;
    float pb[8], px[8];
    sc_unpack8(*(const uint4*)(pr + cb), pb);
    sc_unpack8(*(const uint4*)(pr + cx), px);
#pragma unroll
    for (int e = 0; e < 8; ++e) win[t][e] = pb[e] * px[e];
  }
  for (int rb = r0; rb < r0 + BODY_ROWS && rb < T; rb += RB) {
    uint4 vb[RB], vx[RB], vc[RB];
    int first[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      const int r = rb + i < T ? rb + i : T - 1;
      const bf16* row = bcx + (size_t)r * ld;
      vb[i] = *(const uint4*)(row + cb); vx[i] = *(const uint4*)(row + cx); vc[i] = *(const uint4*)(row + cc);
      first[i] = row_item[r];
    }
#pragma unroll
    for (int i = 0; i < RB; ++i) first[i] = item_start[first[i]];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      const int r = rb + i;
      if (r >= T) break;
      float b[8], x[8], bx[8], conv[8];
      sc_unpack8(vb[i], b);
      sc_unpack8(vx[i], x);
#pragma unroll
      for (int e = 0; e < 8; ++e) { bx[e] = b[e] * x[e]; conv[e] = bx[e] * wt[H][e]; }
#pragma unroll
      for (int t = 0; t < H; ++t) {
#pragma unroll
        for (int e = 0; e < 8; ++e) conv[e] = fmaf(win[t][e], wt[t][e], conv[e]);
      }
#pragma unroll
      for (int t = 0; t + 1 < H; ++t) {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[t][e] = win[t + 1][e];
      }
      if (H > 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[H - 1][e] = bx[e];
      }
      if (r - first[i] < H) continue;             // head rows belong to the item's head thread
      float cg[8];
      sc_unpack8(vc[i], cg);
      uint4 o;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(cg[0] * (conv[0] + bias[0]), cg[1] * (conv[1] + bias[1]));
      __nv_bfloat162 p1 = __floats2bfloat162_rn(cg[2] * (conv[2] + bias[2]), cg[3] * (conv[3] + bias[3]));
      __nv_bfloat162 p2 = __floats2bfloat162_rn(cg[4] * (conv[4] + bias[4]), cg[5] * (conv[5] + bias[5]));
      __nv_bfloat162 p3 = __floats2bfloat162_rn(cg[6] * (conv[6] + bias[6]), cg[7] * (conv[7] + bias[7]));
      o.x = *(unsigned*)&p0; o.y = *(unsigned*)&p1; o.z = *(unsigned*)&p2; o.w = *(unsigned*)&p3;
      *(uint4*)(y + (size_t)r * d + c0) = o;
    }
  }
}

template <typename TA, int VLC>
__global__ void shortconv_kernel(const TA* __restrict__ bcx, const float* __restrict__ w,
                                 const float* __restrict__ conv_bias, float* __restrict__ state,
                                 long long slot_stride, const int* __restrict__ item_slot,
                                 const int* __restrict__ item_start, const int* __restrict__ row_item,
                                 TA* __restrict__ y, int T, int n_items, int d, int Lc, int n_body_tiles, int blocked) {
  FELLM_TRACE_SCOPE(TRACE_SHORTCONV);
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  if (VLC > 0 && (int)blockIdx.y < n_body_tiles) {
    pdl_wait(); FELLM_TRACE_WAITED();
    shortconv_body_vec<(VLC > 0 ? VLC : 2)>((const bf16*)bcx, w, conv_bias, item_start, row_item, (bf16*)y, T, d, blocked);
    return;
  }
  if (c >= d) return;
  const int H = Lc - 1;
  float wt[MAX_LC];
#pragma unroll
  for (int t = 0; t < MAX_LC; ++t) wt[t] = t < Lc ? w[(size_t)c * Lc + t] : 0.f;      // weights: before the wait
  const float wlast = w[(size_t)c * Lc + (Lc - 1)];
  float bias = conv_bias ? conv_bias[c] : 0.f;
  pdl_wait(); FELLM_TRACE_WAITED();
  const size_t ld = (size_t)3 * d;
  const int cb = sc_col(0, c, d, blocked), cc = sc_col(1, c, d, blocked), cx = sc_col(2, c, d, blocked);

  if ((int)blockIdx.y < n_body_tiles) {
    int r0 = blockIdx.y * BODY_ROWS;
    for (int r = r0; r < r0 + BODY_ROWS && r < T; ++r) {
      int j = r - item_start[row_item[r]];
      if (j < H) continue;                       // head rows belong to the item's head thread
      const TA* row = bcx + (size_t)r * ld;
      float bx = to_f(row[cb]) * to_f(row[cx]);
      float conv = bx * wlast;
#pragma unroll
      for (int t = 0; t < MAX_LC - 1; ++t) {
        if (t < H) {
          const TA* pr = bcx + (size_t)(r - H + t) * ld;
          float pbx = to_f(pr[cb]) * to_f(pr[cx]);
          conv = fmaf(pbx, wt[t], conv);
        }
      }
      y[(size_t)r * d + c] = from_f<TA>(to_f(row[cc]) * (conv + bias));
    }
    return;
  }

  int item = blockIdx.y - n_body_tiles;
  if (item >= n_items) return;
  int start = item_start[item], n = item_start[item + 1] - start;
  float* st = state + (size_t)item_slot[item] * slot_stride;       // [Lc-1, d], index 0 oldest
  float hist[MAX_LC - 1];
#pragma unroll
  for (int t = 0; t < MAX_LC - 1; ++t) hist[t] = t < H ? st[(size_t)t * d + c] : 0.f;
  int n_head = n < H ? n : H;
  for (int j = 0; j < n_head; ++j) {
    const TA* row = bcx + (size_t)(start + j) * ld;
    float bx = to_f(row[cb]) * to_f(row[cx]);
    float conv = bx * wlast;
#pragma unroll
    for (int t = 0; t < MAX_LC - 1; ++t)
      if (t < H) conv = fmaf(hist[t], wt[t], conv);
    y[(size_t)(start + j) * d + c] = from_f<TA>(to_f(row[cc]) * (conv + bias));
#pragma unroll
    for (int t = 0; t < MAX_LC - 2; ++t) hist[t] = hist[t + 1];
    // append at index H-1 (the loop above shifted one too far for t >= H-1, fixed here)
#pragma unroll
    for (int t = 0; t < MAX_LC - 1; ++t)
      if (t == H - 1) hist[t] = bx;
  }
  if (n > H) {        // the state is the last Lc-1 products of the portion
#pragma unroll
    for (int t = 0; t < MAX_LC - 1; ++t) {
      if (t < H) {
        const TA* pr = bcx + (size_t)(start + n - H + t) * ld;
        hist[t] = to_f(pr[cb]) * to_f(pr[cx]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MAX_LC - 1; ++t)
    if (t < H) st[(size_t)t * d + c] = hist[t];
}

// bcx [T, 3d] (B | C | X thirds; or, blocked, [B16 | C16 | X16] per 16 channels), w [d, Lc] float32 (tap Lc-1 multiplies the current token),
// conv_bias [d] or null, state: base of this layer's slots, slot_stride floats between slots.
static int conv_class(int rows) {
  static int from = -1;
  if (from < 0) { const char* e = getenv("FELLM_B200_NORM_PDL_ROWS"); from = e ? atoi(e) : 17; }
  return rows >= from ? 1 : 2;
}

FELLM_API int fellm_shortconv(const void* bcx, int is_bf16, const float* w, const float* conv_bias,
                              float* state, long long slot_stride, const int* item_slot,
                              const int* item_start, const int* row_item, void* y, int T, int n_items,
                              int d, int Lc, int all_single, int blocked, cudaStream_t stream) {
  if (T <= 0 || n_items <= 0) return 0;
  if (blocked && (d % 16)) return FELLM_ERR_SIZE;
  if (Lc < 2 || Lc > MAX_LC) return FELLM_ERR_SIZE;
  if (!bcx || !w || !state || !y) return FELLM_ERR_ARG;
  int threads = d >= 128 ? 128 : 64;
  int n_body = all_single ? 0 : ceil_div(T, BODY_ROWS);    // every item has one token: heads only
  const int gx = ceil_div(d, threads);
  if (is_bf16 && d % 8 == 0 && n_body > 0 && Lc <= 5) {
    // vectorised body: a thread takes 8 channels of a tile of BODY_ROWS rows; a grid row holds
    // (gx * threads) / (d / 8) >= 8 such tiles
    const int tiles_per_y = (gx * threads) / (d / 8);
    n_body = ceil_div(n_body, tiles_per_y);
    dim3 grid(gx, n_body + n_items);
#define SC_VEC(LC_) launch_k_class(conv_class(T), shortconv_kernel<bf16, LC_>, grid, dim3(threads), 0, stream, 1, (const bf16*)bcx, w, conv_bias, state, \
                    slot_stride, item_slot, item_start, row_item, (bf16*)y, T, n_items, d, Lc, n_body, blocked)
    switch (Lc) {
      case 2: return SC_VEC(2);
      case 3: return SC_VEC(3);
      case 4: return SC_VEC(4);
      default: return SC_VEC(5);
    }
#undef SC_VEC
  }
  dim3 grid(gx, n_body + n_items);
  if (is_bf16)
    return launch_k_class(conv_class(T), shortconv_kernel<bf16, 0>, grid, dim3(threads), 0, stream, 1, (const bf16*)bcx, w, conv_bias, state,
                    slot_stride, item_slot, item_start, row_item, (bf16*)y, T, n_items, d, Lc, n_body, blocked);
  return launch_k_class(conv_class(T), shortconv_kernel<float, 0>, grid, dim3(threads), 0, stream, 1, (const float*)bcx, w, conv_bias, state,
                  slot_stride, item_slot, item_start, row_item, (float*)y, T, n_items, d, Lc, n_body, blocked);
}

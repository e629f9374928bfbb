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

template <typename TA>
__global__ void shortconv_kernel(const TA* __restrict__ bcx, const float* __restrict__ w,
                                 const float* __restrict__ conv_bias, float* __restrict__ state,
                                 long long slot_stride, const int* __restrict__ item_slot,
                                 const int* __restrict__ item_start, const int* __restrict__ row_item,
                                 TA* __restrict__ y, int T, int n_items, int d, int Lc, int n_body_tiles) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  if (c >= d) return;
  const int H = Lc - 1;
  float wt[MAX_LC];
#pragma unroll
  for (int t = 0; t < MAX_LC; ++t) wt[t] = t < Lc ? w[(size_t)c * Lc + t] : 0.f;      // weights: before the wait
  const float wlast = w[(size_t)c * Lc + (Lc - 1)];
  float bias = conv_bias ? conv_bias[c] : 0.f;
  pdl_wait();
  const size_t ld = (size_t)3 * d;

  if ((int)blockIdx.y < n_body_tiles) {
    int r0 = blockIdx.y * BODY_ROWS;
    for (int r = r0; r < r0 + BODY_ROWS && r < T; ++r) {
      int j = r - item_start[row_item[r]];
      if (j < H) continue;                       // head rows belong to the item's head thread
      const TA* row = bcx + (size_t)r * ld;
      float bx = to_f(row[c]) * to_f(row[2 * d + c]);
      float conv = bx * wlast;
#pragma unroll
      for (int t = 0; t < MAX_LC - 1; ++t) {
        if (t < H) {
          const TA* pr = bcx + (size_t)(r - H + t) * ld;
          float pbx = to_f(pr[c]) * to_f(pr[2 * d + c]);
          conv = fmaf(pbx, wt[t], conv);
        }
      }
      y[(size_t)r * d + c] = from_f<TA>(to_f(row[d + c]) * (conv + bias));
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
    float bx = to_f(row[c]) * to_f(row[2 * d + c]);
    float conv = bx * wlast;
#pragma unroll
    for (int t = 0; t < MAX_LC - 1; ++t)
      if (t < H) conv = fmaf(hist[t], wt[t], conv);
    y[(size_t)(start + j) * d + c] = from_f<TA>(to_f(row[d + c]) * (conv + bias));
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
        hist[t] = to_f(pr[c]) * to_f(pr[2 * d + c]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MAX_LC - 1; ++t)
    if (t < H) st[(size_t)t * d + c] = hist[t];
}

// bcx [T, 3d] (B | C | X thirds), w [d, Lc] float32 (tap Lc-1 multiplies the current token),
// conv_bias [d] or null, state: base of this layer's slots, slot_stride floats between slots.
FELLM_API int fellm_shortconv(const void* bcx, int is_bf16, const float* w, const float* conv_bias,
                              float* state, long long slot_stride, const int* item_slot,
                              const int* item_start, const int* row_item, void* y, int T, int n_items,
                              int d, int Lc, int all_single, cudaStream_t stream) {
  if (T <= 0 || n_items <= 0) return 0;
  if (Lc < 2 || Lc > MAX_LC) return FELLM_ERR_SIZE;
  if (!bcx || !w || !state || !y) return FELLM_ERR_ARG;
  int threads = d >= 128 ? 128 : 64;
  int n_body = all_single ? 0 : ceil_div(T, BODY_ROWS);    // every item has one token: heads only
  dim3 grid(ceil_div(d, threads), n_body + n_items);
  if (is_bf16)
    return launch_k(shortconv_kernel<bf16>, grid, dim3(threads), 0, stream, 1, (const bf16*)bcx, w, conv_bias, state,
                    slot_stride, item_slot, item_start, row_item, (bf16*)y, T, n_items, d, Lc, n_body);
  return launch_k(shortconv_kernel<float>, grid, dim3(threads), 0, stream, 1, (const float*)bcx, w, conv_bias, state,
                  slot_stride, item_slot, item_start, row_item, (float*)y, T, n_items, d, Lc, n_body);
}

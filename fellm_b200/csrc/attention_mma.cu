// Causal GQA attention over the paged cache on tensor cores (mma.sync.m16n8k16, ldmatrix,
// cp.async), bfloat16 queries and cache, float32 softmax and sums; compiled for one head size
// (-DHD=...).  Two kernels share one inner step ("a 16-row block of queries against a tile of
// keys in shared memory"):
//
//  * prefill: portions of prompts (and any mix of item lengths).  A CTA takes one item, one kv
//    head and a block of tokens; its 64 query rows are (token, head of the kv head's group), so K
//    and V are read once for all H/G heads.  Key tiles of 64 go through a two-stage cp.async
//    ring shared by the CTA's four warps.
//  * decode: one token per item against thousands of keys, bound by reading K and V once.  A CTA
//    takes one row, one kv head and one range of keys ("split-KV"); its rows are the H/G heads of
//    the group; each warp streams its own 16-key tiles through its own cp.async ring.  Partial
//    (m, l, acc) of the ranges go to a scratch buffer; the CTA that finishes last for a (row, kv
//    head) merges them in range order.
//
// Formulas: crates/fellm-plugin-abi/src/attention_provider.rs:175-237 (scores scaled by
// 1/sqrt(hd), online softmax with m, l and rescaling, out = acc / l).  FeLLM's kernels:
// attention_fa2_prefill_paged (plugins/cuda_kernels/src/oxide_kernels.rs:4673, one warp per query
// row), attention_fa2_decode_paged (5107, one block per head over all keys).
#include <cuda.h>

#include <mutex>

#include "common.cuh"

#ifndef HD
#define HD 64
#endif
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size: a multiple of 16 in 16..256");

constexpr int CPR = HD / 8;                         // 16-byte chunks per row
constexpr bool SWZ = (CPR % 8 == 0);                // rows of whole 128-byte lines: XOR swizzle
constexpr int ROWB = HD * 2 + (SWZ ? 0 : 16);       // else 16 bytes of padding spread the banks
constexpr int KS = HD / 16;                         // k16 steps over the head size
constexpr int DN = HD / 8;                          // n8 tiles over the head size

__device__ __forceinline__ int tile_off(int row, int chunk) {
  return row * ROWB + ((SWZ ? (chunk ^ (row & 7)) : chunk) << 4);
}
__device__ __forceinline__ void cp_async16(unsigned smem_addr, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem));
}
__device__ __forceinline__ void st_shared_zero16(unsigned smem_addr) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(smem_addr), "r"(0u));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(unsigned* r, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned* r, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(unsigned*)&v;
}

// One 16-row block of queries (fragments qf) against NKT*8 keys staged at k_s / v_s (shared-memory
// addresses of [keys][ROWB] tiles).  Thread (g = lane/4, c = lane%4) owns rows g and g+8; a key at
// tile index i (absolute index key0 + i) counts for row r iff lo[r] <= key0 + i <= hi[r].
// m, l: running maximum (log2 domain) and this thread's share of the running sum per row.
template <int NKT, bool MASKED = true>
__device__ __forceinline__ void attend_tile(const unsigned (&qf)[KS][4], unsigned k_s, unsigned v_s, int key0,
                                            const int (&lo)[2], const int (&hi)[2], float scale_log2,
                                            float (&o)[DN][4], float (&m)[2], float (&l)[2], int lane) {
  const int c = lane & 3;
  float s[NKT][4];
#pragma unroll
  for (int n = 0; n < NKT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
  // S = Q K^T: matrices of one ldmatrix.x4 = (keys 0-7, k lo) (keys 0-7, k hi) (keys 8-15, k lo) (keys 8-15, k hi)
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int np = 0; np < NKT / 2; ++np) {
      int row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
      int chunk = ks * 2 + ((lane >> 3) & 1);
      unsigned r[4];
      ldsm_x4(r, k_s + tile_off(row, chunk));
      mma16816(s[2 * np], qf[ks], r[0], r[1]);
      mma16816(s[2 * np + 1], qf[ks], r[2], r[3]);
    }
  }
  // scale, mask, running maximum
  float mx[2] = {m[0], m[1]};
#pragma unroll
  for (int n = 0; n < NKT; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int key = key0 + n * 8 + 2 * c + (e & 1);
      int r = e >> 1;
      float v = (!MASKED || (key >= lo[r] && key <= hi[r])) ? s[n][e] * scale_log2 : -INFINITY;
      s[n][e] = v;
      mx[r] = fmaxf(mx[r], v);
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  float corr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    corr[r] = (mx[r] == -INFINITY) ? 1.f : exp2f(m[r] - mx[r]);       // nothing seen yet: keep the zeros
    m[r] = mx[r];
    l[r] *= corr[r];
  }
#pragma unroll
  for (int d = 0; d < DN; ++d) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
#pragma unroll
  for (int n = 0; n < NKT; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int r = e >> 1;
      float p = (mx[r] == -INFINITY) ? 0.f : exp2f(s[n][e] - mx[r]);
      s[n][e] = p;
      l[r] += p;
    }
  }
  // O += P V: P's accumulators are the A fragments; V^T comes from ldmatrix.trans:
  // (keys 0-7, dims lo) (keys 8-15, dims lo) (keys 0-7, dims hi) (keys 8-15, dims hi)
#pragma unroll
  for (int j = 0; j < NKT / 2; ++j) {
    unsigned a[4] = {pack_bf16(s[2 * j][0], s[2 * j][1]), pack_bf16(s[2 * j][2], s[2 * j][3]),
                     pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]), pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3])};
#pragma unroll
    for (int dn = 0; dn < DN / 2; ++dn) {
      int row = j * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      int chunk = dn * 2 + (lane >> 4);
      unsigned r[4];
      ldsm_x4_trans(r, v_s + tile_off(row, chunk));
      mma16816(o[2 * dn], a, r[0], r[1]);
      mma16816(o[2 * dn + 1], a, r[2], r[3]);
    }
  }
}

// Query fragments of a 16-row block: row_ptr(i) gives the address of row i's HD elements (null:
// a padding row of zeros).
template <typename F>
__device__ __forceinline__ void load_q(unsigned (&qf)[KS][4], F row_ptr, int lane) {
  const int g = lane >> 2, c = lane & 3;
  const bf16* r0 = row_ptr(g);
  const bf16* r1 = row_ptr(g + 8);
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qf[ks][0] = r0 ? *(const unsigned*)(r0 + ks * 16 + 2 * c) : 0u;
    qf[ks][1] = r1 ? *(const unsigned*)(r1 + ks * 16 + 2 * c) : 0u;
    qf[ks][2] = r0 ? *(const unsigned*)(r0 + ks * 16 + 8 + 2 * c) : 0u;
    qf[ks][3] = r1 ? *(const unsigned*)(r1 + ks * 16 + 8 + 2 * c) : 0u;
  }
}

// ---- keys as the MMA's rows (decode, up to 8 heads a kv head) ----
// With one query row a head, S = Q K^T fills 2 of the MMA's 16 rows.  Turned round, S^T = K Q^T has 16 KEYS as the
// rows and the (up to 8) heads as the 8 columns: half the MMAs, half the scores and exponentials a lane, half the
// output registers (O^T[dim][head] = V^T P^T).  Thread (g = lane/4, c = lane%4) owns keys g and g+8 of a block of
// 16 and heads 2c and 2c+1; P^T becomes the B operand by movmatrix (an 8x8 transpose across the warp).
__device__ __forceinline__ unsigned movmatrix_trans(unsigned x) {
  unsigned y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}
// Query fragments as the B operand: lane (g, c) holds head g's dims ks*16 + 2c, +1 and ks*16 + 8 + 2c, +1.
template <typename F>
__device__ __forceinline__ void load_q_as_b(unsigned (&qb)[KS][2], F row_ptr, int lane) {
  const int g = lane >> 2, c = lane & 3;
  const bf16* r = row_ptr(g);
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qb[ks][0] = r ? *(const unsigned*)(r + ks * 16 + 2 * c) : 0u;
    qb[ks][1] = r ? *(const unsigned*)(r + ks * 16 + 8 + 2 * c) : 0u;
  }
}
// NKT*8 keys at k_s / v_s against the heads in qb; a key counts iff lo <= key0 + i <= hi.  ot[dm] = O^T of dims
// dm*16 + g (elements 0, 1: heads 2c, 2c+1) and dm*16 + g + 8 (elements 2, 3); m, l per head 2c, 2c+1 (l: this
// thread's keys only).
template <int NKT, bool MASKED>
__device__ __forceinline__ void attend_tile_keys_as_rows(const unsigned (&qb)[KS][2], unsigned k_s, unsigned v_s, int key0,
                                                         int lo, int hi, float scale_log2, float (&ot)[HD / 16][4],
                                                         float (&m)[2], float (&l)[2], int lane) {
  constexpr int KB = NKT / 2;                            // blocks of 16 keys
  const int g = lane >> 2;
  float s[KB][4];
#pragma unroll
  for (int b = 0; b < KB; ++b) { s[b][0] = s[b][1] = s[b][2] = s[b][3] = 0.f; }
  // S^T = K Q^T: one ldmatrix.x4 = (keys 0-7, k lo) (keys 8-15, k lo) (keys 0-7, k hi) (keys 8-15, k hi)
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int b = 0; b < KB; ++b) {
      const int row = b * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = ks * 2 + (lane >> 4);
      unsigned r[4];
      ldsm_x4(r, k_s + tile_off(row, chunk));
      mma16816(s[b], r, qb[ks][0], qb[ks][1]);
    }
  }
  float mx[2] = {m[0], m[1]};
#pragma unroll
  for (int b = 0; b < KB; ++b) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + b * 16 + g + ((e >> 1) << 3);
      const float v = (!MASKED || (key >= lo && key <= hi)) ? s[b][e] * scale_log2 : -INFINITY;
      s[b][e] = v;
      mx[e & 1] = fmaxf(mx[e & 1], v);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
  }
  float corr[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    corr[h] = (mx[h] == -INFINITY) ? 1.f : exp2f(m[h] - mx[h]);       // nothing seen yet: keep the zeros
    m[h] = mx[h];
    l[h] *= corr[h];
  }
#pragma unroll
  for (int dm = 0; dm < HD / 16; ++dm) { ot[dm][0] *= corr[0]; ot[dm][1] *= corr[1]; ot[dm][2] *= corr[0]; ot[dm][3] *= corr[1]; }
#pragma unroll
  for (int b = 0; b < KB; ++b) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = (mx[e & 1] == -INFINITY) ? 0.f : exp2f(s[b][e] - mx[e & 1]);
      s[b][e] = p;
      l[e & 1] += p;
    }
  }
  // O^T += V^T P^T: V^T's A fragments by ldmatrix.trans = (keys 0-7, dims lo) (keys 0-7, dims hi) (keys 8-15, dims lo)
  // (keys 8-15, dims hi)
#pragma unroll
  for (int b = 0; b < KB; ++b) {
    const unsigned p0 = movmatrix_trans(pack_bf16(s[b][0], s[b][1]));       // keys 2c, 2c+1 of head g
    const unsigned p1 = movmatrix_trans(pack_bf16(s[b][2], s[b][3]));       // keys 2c+8, 2c+9
#pragma unroll
    for (int dm = 0; dm < HD / 16; ++dm) {
      const int row = b * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = dm * 2 + ((lane >> 3) & 1);
      unsigned r[4];
      ldsm_x4_trans(r, v_s + tile_off(row, chunk));
      mma16816(ot[dm], r, p0, p1);
    }
  }
}

struct AttnArgs {
  const bf16* q; const bf16* pool; const int* block_table; const int* positions; const int* row_slot;
  const int* item_start;          // prefill: rows of item i are item_start[i] .. item_start[i+1]
  bf16* out; float* scratch; int* counters;
  int max_pages, T, H, G, page_tokens, layer, layers_in_group, window, split_len, max_splits, n_items;
  float scale_log2;
};

__device__ __forceinline__ const bf16* key_row(const AttnArgs& a, const int* bt, int g, int key) {
  int lp = key / a.page_tokens;
  int page = max(bt[lp], 0);                 // an unmapped entry (-1) must never become an address: page 0 is read instead
  return a.pool + ((((size_t)page * a.layers_in_group + a.layer) * 2) * a.G + g) * ((size_t)a.page_tokens * HD)
         + (size_t)(key - lp * a.page_tokens) * HD;
}

// ------------------------------------------------------------------------------------ prefill
#define PF_WARPS 4
#define PF_TK 64                 // keys per tile
#define PF_STAGES 2

__global__ void __launch_bounds__(PF_WARPS * 32) attention_prefill_kernel(AttnArgs a) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_PREFILL);
  extern __shared__ __align__(128) unsigned char smem[];
  const int item = blockIdx.z, g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, c = lane & 3;
  const int R = a.H / a.G;
  const int tokb = max(1, (PF_WARPS * 16) / R);               // tokens per CTA
  pdl_launch_dependents();
  const int row_begin = a.item_start[item], n_rows = a.item_start[item + 1] - row_begin;
  const int n_blocks = (n_rows + tokb - 1) / tokb;
  if ((int)blockIdx.x >= (n_blocks + 1) / 2) return;
  const int item_pos0 = a.positions[row_begin];
  const int* bt = a.block_table + (size_t)a.row_slot[row_begin] * a.max_pages;
  pdl_wait(); FELLM_TRACE_WAITED();
  const unsigned s_base = (unsigned)__cvta_generic_to_shared(smem);
  constexpr int TILE_B = PF_TK * ROWB;                         // bytes of one K (or V) tile

  // Causal work grows with the block's position: a CTA takes block bx and then its mirror
  // n_blocks-1-bx, so that every CTA of an item has the same number of key tiles to go through.
  for (int pass = 0; pass < 2; ++pass) {
    const int blk = pass == 0 ? (int)blockIdx.x : n_blocks - 1 - (int)blockIdx.x;
    if (pass == 1 && blk <= (int)blockIdx.x) break;
    const int tok0 = blk * tokb;
    const int n_tok = min(tokb, n_rows - tok0);
    const int pos0 = item_pos0 + tok0;                         // position of the block's first token

    // this thread's two rows: (token, head of the group)
    int tok[2], hr[2], lo[2], hi[2];
    bool valid[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int rho = warp * 16 + gq + 8 * r;
      tok[r] = rho / R; hr[r] = rho - tok[r] * R;
      valid[r] = tok[r] < n_tok;
      int pos = pos0 + tok[r];
      hi[r] = valid[r] ? pos : -1;
      lo[r] = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
      if (!valid[r]) lo[r] = 1 << 30;
    }
    unsigned qf[KS][4];
    load_q(qf, [&](int i) -> const bf16* {
      int rho = warp * 16 + i; int t = rho / R, h = rho - t * R;
      return t < n_tok ? a.q + ((size_t)(row_begin + tok0 + t) * a.H + g * R + h) * HD : nullptr;
    }, lane);

    float o[DN][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DN; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

    // keys of the whole block: from the first token's window start to the last token's position
    const int k_first = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;
    const int k_last = pos0 + n_tok - 1;
    const int n_tiles = (k_last - k_first) / PF_TK + 1;
    auto issue = [&](int j) {
      if (j < n_tiles) {
        unsigned ks = s_base + (j % PF_STAGES) * 2 * TILE_B, vs = ks + TILE_B;
        int key0 = k_first + j * PF_TK;
        for (int i = threadIdx.x; i < PF_TK * CPR; i += PF_WARPS * 32) {
          int row = i / CPR, ch = i - row * CPR;
          int key = key0 + row;
          if (key <= k_last) {
            const bf16* kp = key_row(a, bt, g, key) + ch * 8;
            cp_async16(ks + tile_off(row, ch), kp);
            cp_async16(vs + tile_off(row, ch), kp + (size_t)a.G * a.page_tokens * HD);
          } else {                       // past the last key: zeros, so that 0 * V stays 0
            st_shared_zero16(ks + tile_off(row, ch));
            st_shared_zero16(vs + tile_off(row, ch));
          }
        }
      }
      cp_async_commit();
    };
    __syncthreads();                                           // the pass before is done with the stages
    issue(0);
    for (int j = 0; j < n_tiles; ++j) {
      issue(j + 1);
      cp_async_wait<1>();
      __syncthreads();
      unsigned ks = s_base + (j % PF_STAGES) * 2 * TILE_B, vs = ks + TILE_B;
      int key0 = k_first + j * PF_TK;
      // a warp whose rows all end before this tile has nothing to add (warp-uniform test)
      int warp_hi = pos0 + min(n_tok - 1, (warp * 16 + 15) / R);
      if (key0 <= warp_hi && warp * 16 < n_tok * R)
        attend_tile<PF_TK / 8>(qf, ks, vs, key0, lo, hi, a.scale_log2, o, m, l, lane);
      __syncthreads();                                         // the stage is refilled by the next issue
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      if (!valid[r]) continue;
      float inv = 1.0f / l[r];
      bf16* dst = a.out + ((size_t)(row_begin + tok0 + tok[r]) * a.H + g * R + hr[r]) * HD;
#pragma unroll
      for (int d = 0; d < DN; ++d)
        *(unsigned*)(dst + d * 8 + 2 * c) = pack_bf16(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------ decode
#define DC_WARPS 4
#define DC_TK 16                 // keys per warp tile; with three stages a CTA's rings take 48 KB at head size 64:
                                 // four CTAs per SM, so that a decode batch's CTAs fit one wave
#define DC_STAGES 3
#define DC_MAX_PAGES 256

// The warps of a decode CTA hold partial results (o, m, l) for the same 16-row block of heads over
// different keys: they are combined through `merge` ([warp][16][HD + 2] floats of shared memory that
// no warp reads as a key tile any more) into the CTA's result, which goes to `out` when the CTA is the
// only one of its (row, kv head), else into the CTA's record of the scratch buffer.
__device__ __forceinline__ void decode_merge_records(const AttnArgs& a, const float* merge, int t, int g, int r0, int R,
                                                     int split_index, int n_active, float* cta_rec = nullptr);
__device__ __forceinline__ void decode_warps_to_cta(const AttnArgs& a, float (&o)[DN][4], float (&m)[2], float (&l)[2],
                                                    float* merge, int warp, int lane, int t, int g, int r0, int R,
                                                    int split_index, int n_active, float* cta_rec = nullptr) {
  const int gq = lane >> 2, c = lane & 3;
  const int SW = HD + 2;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    float* rec = merge + ((size_t)warp * 16 + gq + 8 * r) * SW;
#pragma unroll
    for (int d = 0; d < DN; ++d) { rec[d * 8 + 2 * c] = o[d][2 * r]; rec[d * 8 + 2 * c + 1] = o[d][2 * r + 1]; }
    if (c == 0) { rec[HD] = m[r]; rec[HD + 1] = l[r]; }
  }
  decode_merge_records(a, merge, t, g, r0, R, split_index, n_active, cta_rec);
}
// The same from the keys-as-rows layout (heads 0..7 only: rows 8..15 of the records are not written and, with R <= 8,
// not read).
__device__ __forceinline__ void decode_warps_to_cta_keys_as_rows(const AttnArgs& a, float (&ot)[HD / 16][4], float (&m)[2],
                                                                 float (&l)[2], float* merge, int warp, int lane, int t,
                                                                 int g, int R, int split_index, int n_active,
                                                                 float* cta_rec = nullptr) {
  const int gq = lane >> 2, c = lane & 3;
  const int SW = HD + 2;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 4);
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 8);
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 16);
    float* rec = merge + ((size_t)warp * 16 + 2 * c + e) * SW;
#pragma unroll
    for (int dm = 0; dm < HD / 16; ++dm) { rec[dm * 16 + gq] = ot[dm][e]; rec[dm * 16 + gq + 8] = ot[dm][2 + e]; }
    if (gq == 0) { rec[HD] = m[e]; rec[HD + 1] = l[e]; }
  }
  decode_merge_records(a, merge, t, g, 0, R, split_index, n_active, cta_rec);
}
// cta_rec: the CTA's record stays in its shared memory ([row][HD + 2] floats) for the cluster's first active CTA to
// read, instead of going to the scratch buffer.
__device__ __forceinline__ void decode_merge_records(const AttnArgs& a, const float* merge, int t, int g, int r0, int R,
                                                     int split_index, int n_active, float* cta_rec) {
  const int SW = HD + 2;
  __syncthreads();
  const int rows_here = min(16, R - r0);
  for (int i = threadIdx.x; i < rows_here * HD; i += DC_WARPS * 32) {
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
    if (n_active == 1) {
      a.out[((size_t)t * a.H + h) * HD + d] = __float2bfloat16_rn(at / lt);
    } else {
      float* rec = cta_rec ? cta_rec + (size_t)(r0 + row) * SW
                           : a.scratch + (((size_t)t * a.H + h) * a.max_splits + split_index) * SW;
      rec[d] = at;
      if (d == 0) { rec[HD] = mx; rec[HD + 1] = lt; }
    }
  }
  __syncthreads();
}

// The last CTA of a (row, kv head) to get here merges the ranges' records in order.
__device__ __forceinline__ void decode_last_cta_merges(const AttnArgs& a, int* sm_last, int t, int g, int R, int n_active) {
  if (n_active == 1) return;
  const int SW = HD + 2;
  __threadfence();                                      // every writer publishes its records ...
  __syncthreads();                                      // ... before thread 0 counts this CTA in
  if (threadIdx.x == 0) {
    int old = atomicAdd(&a.counters[t * a.G + g], 1);
    *sm_last = (old == n_active - 1);
    if (*sm_last) a.counters[t * a.G + g] = 0;          // ready for the next launch
  }
  __syncthreads();
  if (!*sm_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < R * HD; i += DC_WARPS * 32) {
    int r = i / HD, d = i - r * HD;
    int h = g * R + r;
    const float* rec = a.scratch + ((size_t)t * a.H + h) * a.max_splits * SW;
    float mx = -INFINITY;
    for (int j = 0; j < n_active; ++j) mx = fmaxf(mx, rec[(size_t)j * SW + HD]);
    float lt = 0.f, at = 0.f;
    for (int j = 0; j < n_active; ++j) {
      float cj = exp2f(rec[(size_t)j * SW + HD] - mx);
      lt += rec[(size_t)j * SW + HD + 1] * cj;
      at += rec[(size_t)j * SW + d] * cj;
    }
    a.out[((size_t)t * a.H + h) * HD + d] = __float2bfloat16_rn(at / lt);
  }
}

__global__ void __launch_bounds__(DC_WARPS * 32) attention_decode_kernel(AttnArgs a) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_DECODE);
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int sm_pages[DC_MAX_PAGES];
  __shared__ int sm_last;
  const int s = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // positions, slots and block tables are written by copies before the step's kernels, not by a
  // kernel: they may be read before the wait
  const int pos = a.positions[t];
  const int kb = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  // a launch with fewer key ranges than the longest row has (max_splits * split_len <= pos): the
  // last range takes every key behind it, so that the result stays right (only slower)
  const int s_end = (int)gridDim.x - 1;
  const int s_lo = min(kb / a.split_len, s_end), s_hi = min(pos / a.split_len, s_end);
  pdl_launch_dependents();
  if (s < s_lo || s > s_hi) return;
  const int n_active = s_hi - s_lo + 1;
  const int k0 = max(kb, s * a.split_len), k1 = s == s_end ? pos + 1 : min(pos + 1, (s + 1) * a.split_len);
  const int R = a.H / a.G;
  const int* bt = a.block_table + (size_t)a.row_slot[t] * a.max_pages;
  const int pg0 = k0 / a.page_tokens, n_pg = (k1 - 1) / a.page_tokens - pg0 + 1;
  const bool pages_in_smem = n_pg <= DC_MAX_PAGES;
  if (pages_in_smem)
    for (int i = threadIdx.x; i < n_pg; i += DC_WARPS * 32) sm_pages[i] = bt[pg0 + i];
  pdl_wait(); FELLM_TRACE_WAITED();
  __syncthreads();
  constexpr int TILE_B = DC_TK * ROWB;
  const unsigned ring = (unsigned)__cvta_generic_to_shared(smem) + warp * DC_STAGES * 2 * TILE_B;
  float* merge = (float*)smem;       // [warp][16][HD + 2], over the rings once every warp is done with them
  const int cta_step = DC_WARPS * DC_TK;
  const int n_tiles = (k1 - k0 - warp * DC_TK + cta_step - 1) / cta_step;          // may be <= 0
  const size_t page_elems = (size_t)a.page_tokens * HD;
  auto issue = [&](int j) {
    if (j < n_tiles) {
      unsigned ks = ring + (j % DC_STAGES) * 2 * TILE_B, vs = ks + TILE_B;
      int key0 = k0 + (j * DC_WARPS + warp) * DC_TK;
      for (int i = lane; i < DC_TK * CPR; i += 32) {
        int row = i / CPR, ch = i - row * CPR;
        int key = key0 + row;
        if (key < k1) {
          int lp = key / a.page_tokens;
          int page = max(pages_in_smem ? sm_pages[lp - pg0] : bt[lp], 0);      // never an address below the pool
          const bf16* kp = a.pool + ((((size_t)page * a.layers_in_group + a.layer) * 2) * a.G + g) * page_elems
                           + (size_t)(key - lp * a.page_tokens) * HD + ch * 8;
          cp_async16(ks + tile_off(row, ch), kp);
          cp_async16(vs + tile_off(row, ch), kp + (size_t)a.G * page_elems);
        } else {                       // past the range: zeros, so that 0 * V stays 0
          st_shared_zero16(ks + tile_off(row, ch));
          st_shared_zero16(vs + tile_off(row, ch));
        }
      }
    }
    cp_async_commit();
  };

  for (int r0 = 0; r0 < R; r0 += 16) {                         // groups of more than 16 heads: in blocks
#pragma unroll
    for (int j = 0; j < DC_STAGES - 1; ++j) issue(j);
    unsigned qf[KS][4];
    load_q(qf, [&](int i) -> const bf16* {
      return r0 + i < R ? a.q + ((size_t)t * a.H + g * R + r0 + i) * HD : nullptr;
    }, lane);
    float o[DN][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DN; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    int lo[2] = {k0, k0}, hi[2] = {k1 - 1, k1 - 1};
    for (int j = 0; j < n_tiles; ++j) {
      issue(j + DC_STAGES - 1);
      cp_async_wait<DC_STAGES - 1>();
      __syncwarp();
      unsigned ks = ring + (j % DC_STAGES) * 2 * TILE_B, vs = ks + TILE_B;
      attend_tile<DC_TK / 8>(qf, ks, vs, k0 + (j * DC_WARPS + warp) * DC_TK, lo, hi, a.scale_log2, o, m, l, lane);
      __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();                                           // every warp has left its ring
    decode_warps_to_cta(a, o, m, l, merge, warp, lane, t, g, r0, R, s - s_lo, n_active);
    __syncthreads();
  }
  decode_last_cta_merges(a, &sm_last, t, g, R, n_active);
}

// ------------------------------------------------------------------------------------ decode, TMA
// Head size 64 and pages of 64 tokens: the [64 keys, 64 dims] tile of one kv head of one page is 8 KB
// of contiguous cache, 128 bytes a row, so ONE cp.async.bulk.tensor with the 128-byte swizzle brings
// it in the layout attend_tile() reads (16-byte chunk ^ (row & 7)).  A warp takes every fourth page
// of the CTA's key range, in halves of 32 keys through two stages: one lane asks for a half page's
// K and V tiles, the warp waits on the stage's mbarrier, attends to the 32 keys while the other
// half is on its way, and asks for the half after that.  No address arithmetic per 16 bytes:
// a third of the instructions of the cp.async kernel, which stays for other head and page sizes.
// Waits are bounded (a second): a warp that gives up sets *status = 301 and the CTA finishes with
// what it has.
#if HD == 64
#define DT_PT 64
#define DT_HALF 32                     // keys per tile: half a page, so that a warp has two tiles in flight
#define DT_TILE_B (DT_HALF * 128)
#define DT_WAIT_NS 1000000000ull

__device__ __forceinline__ void at_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void at_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool at_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool at_mbar_wait(unsigned bar, unsigned parity) {
  if (at_mbar_try(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
  for (unsigned i = 0; i < (1u << 26); ++i) {
    if (at_mbar_try(bar, parity)) return true;
    if ((i & 63) == 63) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
      if (t1 - t0 > DT_WAIT_NS) break;
    }
  }
  return false;
}
__device__ __forceinline__ void at_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

// The step's own q, k, v taken straight from the QKV product's output [T, (H+2G)*64], so that the
// per-head RMSNorm, the rotation and the write of k and v into the cache need no kernel of their
// own (formulas: qk_rope_write.cu).  qkv null: q comes normed and rotated in AttnArgs::q.
struct DecodeFuse {
  const bf16* qkv; const float* q_w; const float* k_w; const float* inv_freq;
  float eps; int pairing;
};

// One head of 64 elements by a warp, lane l holding elements 2l and 2l+1: RMSNorm (if w), rotation
// by pos (if inv_freq) on pairs (2i, 2i+1) (pairing 0) or (i, i+32) (pairing 1).  What does not
// depend on the kernel in front (the angles' sines and cosines, the norm weights) is worked out by
// rope_coeffs()/norm_weights() before the wait for it.
struct RopeCoeffs { float s0, c0, s1, c1; };
__device__ __forceinline__ RopeCoeffs rope_coeffs(const float* inv_freq, int pairing, int pos, int lane) {
  RopeCoeffs r = {0.f, 1.f, 0.f, 1.f};
  if (inv_freq) {
    if (pairing == 0) {
      sincosf((float)pos * inv_freq[lane], &r.s0, &r.c0);
    } else {
      const int p0 = (2 * lane) & 31;
      sincosf((float)pos * inv_freq[p0], &r.s0, &r.c0);
      sincosf((float)pos * inv_freq[p0 + 1], &r.s1, &r.c1);
    }
  }
  return r;
}
__device__ __forceinline__ float2 norm_weights(const float* w, int lane) {
  return w ? make_float2(w[2 * lane], w[2 * lane + 1]) : make_float2(1.f, 1.f);
}
__device__ __forceinline__ float2 norm_rope_head64(const bf16* src, bool norm, float2 w, float eps, bool rotate,
                                                   int pairing, const RopeCoeffs& rc, int lane) {
  float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(src + 2 * lane));
  if (norm) {
    float ss = fmaf(v.x, v.x, v.y * v.y);
    ss = warp_sum(ss);
    const float sc = 1.0f / sqrtf(ss / 64.0f + eps);
    v.x = (v.x * sc) * w.x;
    v.y = (v.y * sc) * w.y;
  }
  if (rotate) {
    if (pairing == 0) {
      const float x = v.x, y = v.y;
      v.x = x * rc.c0 - y * rc.s0; v.y = x * rc.s0 + y * rc.c0;
    } else {
      const float ox = __shfl_xor_sync(0xffffffffu, v.x, 16), oy = __shfl_xor_sync(0xffffffffu, v.y, 16);
      if (lane < 16) { v.x = v.x * rc.c0 - ox * rc.s0; v.y = v.y * rc.c1 - oy * rc.s1; }      // first of the pair: a*c - b*s
      else { v.x = ox * rc.s0 + v.x * rc.c0; v.y = oy * rc.s1 + v.y * rc.c1; }                // second: a*s + b*c
    }
  }
  return v;
}

// NS: half-page stages a warp keeps in flight (2: 64 KB a CTA, three CTAs to an SM; 3: 96 KB, two; 4: 128 KB, one).
__device__ __forceinline__ float ld_cluster_f32(unsigned addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned mapa_cta(unsigned smem_addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {       // every thread of every CTA of the cluster, the same number of times
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// KR: keys as the MMA's rows (up to 8 heads a kv head).  CL: the key ranges of a (row, kv head) are the CTAs of
// one cluster (up to 8): their records stay in shared memory and the first active one adds them up in range order
// through distributed shared memory, instead of records in a scratch buffer, a fence, a counter and the last CTA
// reading them back from L2.  Every CTA of the cluster, active or not, passes the same two cluster barriers.
template <int NS, bool KR, bool CL>
__global__ void __launch_bounds__(DC_WARPS * 32)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap pool_map, AttnArgs a, DecodeFuse f, int* status) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_DECODE);
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[DC_WARPS * NS];
  __shared__ int sm_pages[DC_MAX_PAGES];
  __shared__ int sm_last;
  __shared__ __align__(16) bf16 q_s[16 * HD];            // fused: the group's heads, normed and rotated
  const int s = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // positions, slots and block tables are written by copies before the step's kernels, not by a
  // kernel: they may be read before the wait
  const int pos = a.positions[t];
  const int kb = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  // a launch with fewer key ranges than the longest row has (max_splits * split_len <= pos): the
  // last range takes every key behind it, so that the result stays right (only slower)
  const int s_end = (int)gridDim.x - 1;
  const int s_lo = min(kb / a.split_len, s_end), s_hi = min(pos / a.split_len, s_end);
  pdl_launch_dependents();
  const bool active = s >= s_lo && s <= s_hi;
  if (!CL && !active) return;
  const int n_active = s_hi - s_lo + 1;
  const int R = a.H / a.G;                              // <= 16 (the launcher checks)
  const unsigned base = ((unsigned)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;      // the swizzle is by address
  float* merge = (float*)(smem_raw + (base - (unsigned)__cvta_generic_to_shared(smem_raw)));  // over the tiles, once the warps are done
  float* cta_rec = CL ? merge + DC_WARPS * 16 * (HD + 2) : nullptr;
  if (active) {
  const int k0 = max(kb, s * a.split_len), k1 = s == s_end ? pos + 1 : min(pos + 1, (s + 1) * a.split_len);
  const int* bt = a.block_table + (size_t)a.row_slot[t] * a.max_pages;
  const int pg0 = k0 / DT_PT, n_pg = (k1 - 1) / DT_PT - pg0 + 1;
  const bool pages_in_smem = n_pg <= DC_MAX_PAGES;
  if (pages_in_smem)
    for (int i = threadIdx.x; i < n_pg; i += DC_WARPS * 32) sm_pages[i] = bt[pg0 + i];
  if (threadIdx.x < DC_WARPS * NS) at_mbar_init((unsigned)__cvta_generic_to_shared(&bars[threadIdx.x]), 1);
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();
  // a warp's NS stages, each the K and the V tile of half a page (32 keys)
  const unsigned stage0 = base + warp * NS * 2 * DT_TILE_B;
  const unsigned bar0 = (unsigned)__cvta_generic_to_shared(&bars[warp * NS]);
  const int my_pages = (n_pg - warp + DC_WARPS - 1) / DC_WARPS;                              // may be <= 0
  const int n_tiles = my_pages > 0 ? my_pages * 2 : 0;
  auto request = [&](int q) {                           // lane 0: K and V of the q-th half page of this warp
    const int lp = pg0 + warp + (q >> 1) * DC_WARPS;
    const int page = pages_in_smem ? sm_pages[lp - pg0] : bt[lp];
    const int row = (((page * a.layers_in_group + a.layer) * 2) * a.G + g) * DT_PT + (q & 1) * DT_HALF;   // < 2^31: the launcher checks
    const unsigned st = stage0 + (q % NS) * 2 * DT_TILE_B, bar = bar0 + (q % NS) * 8;
    at_mbar_expect_tx(bar, 2 * DT_TILE_B);
    at_tma_load_2d(st, &pool_map, 0, row, bar);
    at_tma_load_2d(st + DT_TILE_B, &pool_map, 0, row + a.G * DT_PT, bar);
  };
  // Fused, the kernel before this one (the QKV product) writes nothing of the cache: the first tiles
  // are asked for before the wait, the row of the step's own position being replaced in the tile
  // later anyway.  Not fused, that kernel wrote the step's k and v: after the wait.
  const bool early = f.qkv != nullptr;
  RopeCoeffs rc = {0.f, 1.f, 0.f, 1.f};
  float2 qw = make_float2(1.f, 1.f), kw = qw;
  if (early) {                                              // the angles and the norm weights do not wait either
    rc = rope_coeffs(f.inv_freq, f.pairing, pos, lane);
    qw = norm_weights(f.q_w, lane); kw = norm_weights(f.k_w, lane);
  }
  if (early && lane == 0) {
#pragma unroll
    for (int q = 0; q < NS; ++q) if (q < n_tiles) request(q);
  }
  pdl_wait(); FELLM_TRACE_WAITED();
  const bf16* qkv_row = f.qkv ? f.qkv + (size_t)t * (a.H + 2 * a.G) * HD : nullptr;
  if (qkv_row) {
    for (int i = warp; i < 16; i += DC_WARPS) {
      float2 v = make_float2(0.f, 0.f);
      if (i < R) v = norm_rope_head64(qkv_row + (size_t)(g * R + i) * HD, f.q_w != nullptr, qw, f.eps, f.inv_freq != nullptr, f.pairing, rc, lane);
      *(__nv_bfloat162*)(q_s + i * HD + 2 * lane) = __floats2bfloat162_rn(v.x, v.y);
    }
  }
  __syncthreads();
  if (!early && lane == 0) {
#pragma unroll
    for (int q = 0; q < NS; ++q) if (q < n_tiles) request(q);
  }
  auto q_row = [&](int i) -> const bf16* {
    if (i >= R) return nullptr;
    return qkv_row ? q_s + i * HD : a.q + ((size_t)t * a.H + g * R + i) * HD;
  };
  unsigned qf[KR ? 1 : KS][4], qb[KR ? KS : 1][2];
  float o[KR ? 1 : DN][4], ot[KR ? HD / 16 : 1][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  if constexpr (KR) {
    load_q_as_b(qb, q_row, lane);
#pragma unroll
    for (int d = 0; d < HD / 16; ++d) { ot[d][0] = ot[d][1] = ot[d][2] = ot[d][3] = 0.f; }
  } else {
    load_q(qf, q_row, lane);
#pragma unroll
    for (int d = 0; d < DN; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
  }
  const int lo[2] = {k0, k0}, hi[2] = {k1 - 1, k1 - 1};
  for (int q = 0; q < n_tiles; ++q) {
    const unsigned st = stage0 + (q % NS) * 2 * DT_TILE_B, bar = bar0 + (q % NS) * 8;
    const bool arrived = __all_sync(0xffffffffu, at_mbar_wait(bar, (q / NS) & 1));
    if (q == 0) FELLM_TRACE_MARK(0);
    if (!arrived) {
      if (lane == 0 && status) atomicExch(status, 301);
      break;
    }
    const int key0 = (pg0 + warp + (q >> 1) * DC_WARPS) * DT_PT + (q & 1) * DT_HALF;
    if (qkv_row && s == s_hi && key0 <= pos && pos < key0 + DT_HALF) {
      // fused: this tile holds the step's own position; its k (normed, rotated) and v go into the
      // tile and into the cache page (no other CTA or warp reads this page's tile in this step)
      const int lp = pos / DT_PT;
      const int page = pages_in_smem ? sm_pages[lp - pg0] : bt[lp];
      const float2 kv = norm_rope_head64(qkv_row + (size_t)(a.H + g) * HD, f.k_w != nullptr, kw, f.eps, f.inv_freq != nullptr, f.pairing, rc, lane);
      const __nv_bfloat162 kk = __floats2bfloat162_rn(kv.x, kv.y);
      const __nv_bfloat162 vv = *(const __nv_bfloat162*)(qkv_row + (size_t)(a.H + a.G + g) * HD + 2 * lane);
      const unsigned off = tile_off(pos - key0, (2 * lane) >> 3) + ((2 * lane) & 7) * 2;
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(st + off), "r"(*(const unsigned*)&kk) : "memory");
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(st + DT_TILE_B + off), "r"(*(const unsigned*)&vv) : "memory");
      if (page >= 0) {
        bf16* krow = const_cast<bf16*>(a.pool) + ((((size_t)page * a.layers_in_group + a.layer) * 2 * a.G + g) * DT_PT + (pos - lp * DT_PT)) * HD;
        *(__nv_bfloat162*)(krow + 2 * lane) = kk;
        *(__nv_bfloat162*)(krow + (size_t)a.G * DT_PT * HD + 2 * lane) = vv;
      } else if (lane == 0 && status) {
        atomicExch(status, 302);                          // no page mapped for the step's own position
      }
      __syncwarp();
    }
    if (key0 < k1 && key0 + DT_HALF > k0) {              // else: a half page with no key of the range
      if (key0 + DT_HALF > k1) {
        // rows past the last key hold whatever the page held before: zero the V rows, so that 0 * V is 0
        for (int i = (k1 - key0) * CPR + lane; i < DT_HALF * CPR; i += 32) st_shared_zero16(st + DT_TILE_B + tile_off(i / CPR, i % CPR));
        __syncwarp();
      }
      const bool edge = key0 < k0 || key0 + DT_HALF > k1;
      if constexpr (KR) {
        if (edge) attend_tile_keys_as_rows<DT_HALF / 8, true>(qb, st, st + DT_TILE_B, key0, k0, k1 - 1, a.scale_log2, ot, m, l, lane);
        else attend_tile_keys_as_rows<DT_HALF / 8, false>(qb, st, st + DT_TILE_B, key0, k0, k1 - 1, a.scale_log2, ot, m, l, lane);
      } else {
        if (edge) attend_tile<DT_HALF / 8, true>(qf, st, st + DT_TILE_B, key0, lo, hi, a.scale_log2, o, m, l, lane);
        else attend_tile<DT_HALF / 8, false>(qf, st, st + DT_TILE_B, key0, lo, hi, a.scale_log2, o, m, l, lane);
      }
    }
    __syncwarp();
    if (q + NS < n_tiles) {
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // this warp's reads before the next copy's writes
      if (lane == 0) request(q + NS);
    }
  }
  FELLM_TRACE_MARK(1);
  __syncthreads();                                         // every warp has left its tiles
  if constexpr (KR) decode_warps_to_cta_keys_as_rows(a, ot, m, l, merge, warp, lane, t, g, R, s - s_lo, n_active, cta_rec);
  else decode_warps_to_cta(a, o, m, l, merge, warp, lane, t, g, 0, R, s - s_lo, n_active, cta_rec);
  FELLM_TRACE_MARK(2);
  if constexpr (!CL) decode_last_cta_merges(a, &sm_last, t, g, R, n_active);
  }                                                        // active
  if constexpr (CL) {
    cluster_barrier();                                     // the records of all ranges are written
    if (active && n_active > 1 && s == s_lo) {
      const int SW = HD + 2;
      const unsigned mine = (unsigned)__cvta_generic_to_shared(cta_rec);
      for (int i = threadIdx.x; i < R * HD; i += DC_WARPS * 32) {
        const int r = i / HD, d = i - r * HD;
        float mj[8], lj[8], aj[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < n_active) {
            const unsigned rec = mapa_cta(mine + (unsigned)(r * SW) * 4u, (unsigned)(s_lo + j));
            aj[j] = ld_cluster_f32(rec + d * 4);
            mj[j] = ld_cluster_f32(rec + HD * 4);
            lj[j] = ld_cluster_f32(rec + (HD + 1) * 4);
          } else {
            aj[j] = 0.f; mj[j] = -INFINITY; lj[j] = 0.f;
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, mj[j]);
        float lt = 0.f, at = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float cj = j < n_active ? exp2f(mj[j] - mx) : 0.f;
          lt += lj[j] * cj;
          at += aj[j] * cj;
        }
        a.out[((size_t)t * a.H + g * R + r) * HD + d] = __float2bfloat16_rn(at / lt);
      }
    }
    cluster_barrier();                                     // nobody leaves while its record may be read
  }
}

// ------------------------------------------------------------------------------------ prefill, TMA
// The prefill kernel for head size 64, pages of 64 tokens and no window: a key tile IS a page, so
// one thread brings K and V of a tile with two bulk tensor copies (three stages on mbarriers with
// bounded waits) instead of 128 threads computing an address per 16 bytes, and tiles that every row
// of a warp sees whole skip the masking.  Same sums in the same order as attention_prefill_kernel.
#define PT_STAGES 3
__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap pool_map, AttnArgs a, int* status) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_PREFILL);
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[PT_STAGES];
  __shared__ int sm_fail;
  const int item = blockIdx.z, g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, c = lane & 3;
  const int R = a.H / a.G;
  const int tokb = max(1, (PF_WARPS * 16) / R);               // tokens per CTA
  pdl_launch_dependents();
  const int row_begin = a.item_start[item], n_rows = a.item_start[item + 1] - row_begin;
  const int n_blocks = (n_rows + tokb - 1) / tokb;
  if ((int)blockIdx.x >= (n_blocks + 1) / 2) return;
  const int item_pos0 = a.positions[row_begin];
  const int* bt = a.block_table + (size_t)a.row_slot[row_begin] * a.max_pages;
  if (threadIdx.x < PT_STAGES) at_mbar_init((unsigned)__cvta_generic_to_shared(&bars[threadIdx.x]), 1);
  if (threadIdx.x == 0) sm_fail = 0;
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  pdl_wait(); FELLM_TRACE_WAITED();
  __syncthreads();
  const unsigned s_base = ((unsigned)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  const unsigned bar0 = (unsigned)__cvta_generic_to_shared(&bars[0]);
  constexpr int TILE_B = DT_PT * 128;                          // bytes of one K (or V) tile: a page
  unsigned it_issue = 0, it_use = 0;                           // tiles requested / consumed so far, over both passes

  // Causal work grows with the block's position: a CTA takes block bx and then its mirror
  // n_blocks-1-bx, so that every CTA of an item has the same number of key tiles to go through.
  for (int pass = 0; pass < 2; ++pass) {
    const int blk = pass == 0 ? (int)blockIdx.x : n_blocks - 1 - (int)blockIdx.x;
    if (pass == 1 && blk <= (int)blockIdx.x) break;
    const int tok0 = blk * tokb;
    const int n_tok = min(tokb, n_rows - tok0);
    const int pos0 = item_pos0 + tok0;                         // position of the block's first token
    int tok[2], hr[2], lo[2], hi[2];
    bool valid[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int rho = warp * 16 + gq + 8 * r;
      tok[r] = rho / R; hr[r] = rho - tok[r] * R;
      valid[r] = tok[r] < n_tok;
      hi[r] = valid[r] ? pos0 + tok[r] : -1;
      lo[r] = valid[r] ? 0 : 1 << 30;
    }
    unsigned qf[KS][4];
    load_q(qf, [&](int i) -> const bf16* {
      int rho = warp * 16 + i; int t = rho / R, h = rho - t * R;
      return t < n_tok ? a.q + ((size_t)(row_begin + tok0 + t) * a.H + g * R + h) * HD : nullptr;
    }, lane);
    float o[DN][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DN; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

    const int k_last = pos0 + n_tok - 1;
    const int n_tiles = k_last / DT_PT + 1;                    // pages 0 .. that of the last token
    auto issue = [&](int j) {                                  // thread 0: tile j of this pass = page j
      const unsigned st = s_base + (it_issue % PT_STAGES) * 2 * TILE_B, bar = bar0 + (it_issue % PT_STAGES) * 8;
      const int page = bt[j];
      const int row = (((page * a.layers_in_group + a.layer) * 2) * a.G + g) * DT_PT;      // < 2^31: the launcher checks
      at_mbar_expect_tx(bar, 2 * TILE_B);
      at_tma_load_2d(st, &pool_map, 0, row, bar);
      at_tma_load_2d(st + TILE_B, &pool_map, 0, row + a.G * DT_PT, bar);
      ++it_issue;
    };
    // every warp has left the stages of the pass before (the loop below ends on a barrier)
    if (threadIdx.x == 0) {
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      for (int j = 0; j < PT_STAGES - 1 && j < n_tiles; ++j) issue(j);
    }
    // rows of this warp see a tile whole when it ends at or before the warp's first token
    const bool warp_full = (warp * 16 + 15) < n_tok * R;
    const int warp_first = pos0 + (warp * 16) / R, warp_hi = pos0 + min(n_tok - 1, (warp * 16 + 15) / R);
    bool failed = false;
    for (int j = 0; j < n_tiles; ++j) {
      if (threadIdx.x == 0 && j + PT_STAGES - 1 < n_tiles) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // the reads of tile j-1 before the copy into its stage
        issue(j + PT_STAGES - 1);
      }
      const unsigned st = s_base + (it_use % PT_STAGES) * 2 * TILE_B, bar = bar0 + (it_use % PT_STAGES) * 8;
      if (!at_mbar_wait(bar, (it_use / PT_STAGES) & 1)) { sm_fail = 1; if (status) atomicExch(status, 301); }
      ++it_use;
      const int key0 = j * DT_PT;
      if (key0 + DT_PT > k_last + 1) {
        // rows past the last key hold whatever the page held before: zero the V rows, so that 0 * V is 0
        for (int i = (k_last + 1 - key0) * CPR + threadIdx.x; i < DT_PT * CPR; i += PF_WARPS * 32)
          st_shared_zero16(st + TILE_B + tile_off(i / CPR, i % CPR));
        __syncthreads();
      }
      if (key0 <= warp_hi && warp * 16 < n_tok * R) {
        if (warp_full && key0 + DT_PT - 1 <= warp_first)
          attend_tile<DT_PT / 8, false>(qf, st, st + TILE_B, key0, lo, hi, a.scale_log2, o, m, l, lane);
        else
          attend_tile<DT_PT / 8, true>(qf, st, st + TILE_B, key0, lo, hi, a.scale_log2, o, m, l, lane);
      }
      __syncthreads();                                         // the stage may be refilled; sm_fail is seen by all
      if (sm_fail) { failed = true; break; }
    }
    if (failed) break;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      if (!valid[r]) continue;
      float inv = 1.0f / l[r];
      bf16* dst = a.out + ((size_t)(row_begin + tok0 + tok[r]) * a.H + g * R + hr[r]) * HD;
#pragma unroll
      for (int d = 0; d < DN; ++d)
        *(unsigned*)(dst + d * 8 + 2 * c) = pack_bf16(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
  }
}

// The cache pool as a 2-D tensor [rows of 64 dims]: the map is kept per (pool, rows, rows of a box).
typedef CUresult (*AtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int pool_map_for(const void* pool, long long rows, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static struct { const void* pool; long long rows; int box_rows; CUtensorMap map; } cache[8];
  static int n_cached = 0, next = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_cached; ++i)
    if (cache[i].pool == pool && cache[i].rows == rows && cache[i].box_rows == box_rows) { *out = cache[i].map; return 0; }
  static AtEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return FELLM_ERR_ARG;
    fn = (AtEncodeTiledFn)p;
  }
  cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
  cuuint32_t box[2] = {HD, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  cache[next].pool = pool; cache[next].rows = rows; cache[next].box_rows = box_rows; cache[next].map = m;
  next = (next + 1) % 8;
  if (n_cached < 8) ++n_cached;
  *out = m;
  return 0;
}
#endif

static int fill_args(AttnArgs& a, const void* q, const void* pool, const int* block_table, int max_pages,
                     const int* positions, const int* row_slot, void* out, int T, int H, int G, int hd,
                     int page_tokens, int layer, int layers_in_group, float scale, int window) {
  if (hd != HD) return FELLM_ERR_SIZE;
  if (G < 1 || H % G) return FELLM_ERR_SIZE;
  if (!q || !pool || !block_table || !positions || !row_slot || !out) return FELLM_ERR_ARG;
  a.q = (const bf16*)q; a.pool = (const bf16*)pool; a.block_table = block_table; a.positions = positions;
  a.row_slot = row_slot; a.out = (bf16*)out; a.max_pages = max_pages; a.T = T; a.H = H; a.G = G;
  a.page_tokens = page_tokens; a.layer = layer; a.layers_in_group = layers_in_group; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.item_start = nullptr; a.scratch = nullptr; a.counters = nullptr; a.split_len = 1; a.max_splits = 1; a.n_items = 0;
  return 0;
}

FELLM_API int fellm_attn_head_dim() { return HD; }

// q [T, H, hd], out [T, H*hd]; rows of item i are item_start[i]..item_start[i+1], its positions are
// consecutive from positions[item_start[i]]; max_item_rows: the longest item of the step.
FELLM_API int fellm_attn_prefill_mma(const void* q, const void* pool, const int* block_table, int max_pages,
                                     const int* positions, const int* row_slot, const int* item_start, int n_items,
                                     int max_item_rows, void* out, int T, int H, int G, int hd, int page_tokens,
                                     int layer, int layers_in_group, float scale, int window, cudaStream_t stream) {
  if (T <= 0 || n_items <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, q, pool, block_table, max_pages, positions, row_slot, out, T, H, G, hd, page_tokens, layer,
                    layers_in_group, scale, window);
  if (e) return e;
  if (!item_start) return FELLM_ERR_ARG;
  int R = H / G;
  if (R > PF_WARPS * 16) return FELLM_ERR_SIZE;
  a.item_start = item_start; a.n_items = n_items;
  int tokb = (PF_WARPS * 16) / R; if (tokb < 1) tokb = 1;
  size_t smem = (size_t)PF_STAGES * 2 * PF_TK * ROWB;
  auto kern = attention_prefill_kernel;
  if (smem > 32 * 1024) {        // static shared memory counts against the 48 KB default too
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  return launch_k_class(launch_class_for_rows(T, 0), kern, dim3((ceil_div(max_item_rows, tokb) + 1) / 2, G, n_items), dim3(PF_WARPS * 32), smem, stream, 1, a);
}

// One query row per item.  scratch: float32 [T*H*max_splits*(hd+2)]; counters: int32 [T*G], zero
// before the first launch (the kernel leaves them zero).  max_splits >= ceil(longest context / split_len).
FELLM_API int fellm_attn_decode_mma(const void* q, const void* pool, const int* block_table, int max_pages,
                                    const int* positions, const int* row_slot, void* out, float* scratch,
                                    int* counters, int T, int H, int G, int hd, int page_tokens, int layer,
                                    int layers_in_group, float scale, int window, int split_len, int max_splits,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, q, pool, block_table, max_pages, positions, row_slot, out, T, H, G, hd, page_tokens, layer,
                    layers_in_group, scale, window);
  if (e) return e;
  if (!scratch || !counters || split_len < 1 || max_splits < 1) return FELLM_ERR_ARG;
  a.scratch = scratch; a.counters = counters; a.split_len = split_len; a.max_splits = max_splits;
  size_t ring = (size_t)DC_WARPS * DC_STAGES * 2 * DC_TK * ROWB, mrg = (size_t)DC_WARPS * 16 * (HD + 2) * sizeof(float);
  size_t smem = ring > mrg ? ring : mrg;
  auto kern = attention_decode_kernel;
  if (smem > 32 * 1024) {        // static shared memory counts against the 48 KB default too
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  return launch_k(kern, dim3(max_splits, G, T), dim3(DC_WARPS * 32), smem, stream, 1, a);
}

// The same through the TMA kernel: head size 64, pages of 64 tokens, at most 16 heads per kv head
// (FELLM_ERR_SIZE otherwise: the caller falls back to fellm_attn_decode_mma).  n_pages: pages of the
// pool; status: device int32 set to 301 if a wait ran out.
// qkv non-null: the QKV product's output [T, (H+2G)*64]; the kernel norms (q_w, k_w float32 [64] or null)
// and rotates (inv_freq float32 [32] or null; pairing 0 adjacent / 1 split-half) q and k itself and
// writes k and v into the cache; q is then not read.  status 302: a row's position has no page.
// stages: half pages (32 keys) a warp keeps in flight, 2..4.
FELLM_API int fellm_attn_decode_tma(const void* q, const void* pool, long long n_pages, const int* block_table,
                                    int max_pages, const int* positions, const int* row_slot, void* out,
                                    float* scratch, int* counters, int T, int H, int G, int hd, int page_tokens,
                                    int layer, int layers_in_group, float scale, int window, int split_len,
                                    int max_splits, int* status, const void* qkv, const float* q_w, const float* k_w,
                                    float eps, const float* inv_freq, int pairing, int stages, cudaStream_t stream) {
#if HD == 64
  if (T <= 0) return 0;
  AttnArgs a;
  if (!q) q = qkv;
  int e = fill_args(a, q, pool, block_table, max_pages, positions, row_slot, out, T, H, G, hd, page_tokens, layer,
                    layers_in_group, scale, window);
  if (e) return e;
  if (!scratch || !counters || split_len < 1 || max_splits < 1) return FELLM_ERR_ARG;
  const long long rows = n_pages * layers_in_group * 2 * G * page_tokens;
  if (page_tokens != DT_PT || H / G > 16 || (split_len % DT_PT) || rows >= (1ll << 31) || ((uintptr_t)pool & 15))
    return FELLM_ERR_SIZE;
  a.scratch = scratch; a.counters = counters; a.split_len = split_len; a.max_splits = max_splits;
  CUtensorMap map;
  e = pool_map_for(pool, rows, DT_HALF, &map);
  if (e) return e;
  // stages: half pages a warp keeps in flight, 2 (three CTAs to an SM), 3 or 4 (one CTA to an SM: the few CTAs of
  // a step of one or two requests, which then have most of their keys on the way at once)
  static int ns_env = -1;
  if (ns_env < 0) { const char* ev = getenv("FELLM_B200_DECODE_STAGES"); ns_env = (ev && ev[0] >= '2' && ev[0] <= '4') ? ev[0] - '0' : 0; }
  const int ns = ns_env ? ns_env : (stages >= 2 && stages <= 4 ? stages : 2);
  size_t tiles = (size_t)DC_WARPS * ns * 2 * DT_TILE_B, mrg = (size_t)(DC_WARPS + 1) * 16 * (HD + 2) * sizeof(float);
  size_t smem = (tiles > mrg ? tiles : mrg) + 1024;
  // up to 8 heads a kv head: the keys as the MMA's rows (FELLM_B200_DECODE_KEYS_AS_ROWS=0: the heads, as with more)
  static int kr_env = -1;
  if (kr_env < 0) { const char* ev = getenv("FELLM_B200_DECODE_KEYS_AS_ROWS"); kr_env = (ev && ev[0] == '0') ? 0 : 1; }
  const bool kr = kr_env && H / G <= 8;
  // up to 8 key ranges: they are one cluster and merge through its shared memory (FELLM_B200_DECODE_CLUSTER=0: the
  // scratch buffer and the last CTA, as with more ranges)
  static int cl_env = -1;
  if (cl_env < 0) { const char* ev = getenv("FELLM_B200_DECODE_CLUSTER"); cl_env = (ev && ev[0] == '0') ? 0 : 1; }
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
  }
  // ... where all CTAs are resident at once (measured on B200, 16 layers of width 1024, context 2,050..2,250: batch 8,
  // 6 ranges, 0.374 -> 0.369 ms a step; batch 1, 8 ranges, 0.316 -> 0.310 ms; but batch 64, 1,024 CTAs in pairs over
  // 2.3 waves, 0.826 -> 0.860 ms: a pair waits for a place for both and for the slower of the two)
  const int ctas_per_sm = ns == 2 ? 3 : (ns == 3 ? 2 : 1);
  const bool cl = cl_env && max_splits >= 2 && max_splits <= 8 && (long long)max_splits * G * T <= (long long)n_sm * ctas_per_sm;
  void (*kern)(const CUtensorMap, AttnArgs, DecodeFuse, int*) = nullptr;
#define FELLM_PICK(NS_) \
  kern = kr ? (cl ? attention_decode_tma_kernel<NS_, true, true> : attention_decode_tma_kernel<NS_, true, false>) \
            : (cl ? attention_decode_tma_kernel<NS_, false, true> : attention_decode_tma_kernel<NS_, false, false>)
  if (ns == 2) { FELLM_PICK(2); } else if (ns == 3) { FELLM_PICK(3); } else { FELLM_PICK(4); }
#undef FELLM_PICK
  cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (ce != cudaSuccess) return (int)ce;
  DecodeFuse f;
  f.qkv = (const bf16*)qkv; f.q_w = q_w; f.k_w = k_w; f.inv_freq = inv_freq; f.eps = eps; f.pairing = pairing;
  // fused, the kernel asks for its first tiles before the wait: launched as a programmatic dependent
  // (class 1) it streams the cache under the QKV product (386 against 402 us a step at batch 8;
  // FELLM_B200_ATTN_PDL=0 launches it the ordinary way)
  static int attn_class = -1;
  if (attn_class < 0) { const char* e = getenv("FELLM_B200_ATTN_PDL"); attn_class = (e && e[0] == '0') ? 0 : 1; }
  return launch_k_class(qkv ? attn_class : 0, kern, dim3(max_splits, G, T), dim3(DC_WARPS * 32), smem, stream, cl ? max_splits : 1, map, a, f, status);
#else
  return FELLM_ERR_SIZE;
#endif
}

// The prefill kernel through TMA: head size 64, pages of 64 tokens, no window (FELLM_ERR_SIZE
// otherwise: the caller falls back to fellm_attn_prefill_mma).  status: set to 301 if a wait ran out.
FELLM_API int fellm_attn_prefill_tma(const void* q, const void* pool, long long n_pages, const int* block_table,
                                     int max_pages, const int* positions, const int* row_slot, const int* item_start,
                                     int n_items, int max_item_rows, void* out, int T, int H, int G, int hd,
                                     int page_tokens, int layer, int layers_in_group, float scale, int window,
                                     int* status, cudaStream_t stream) {
#if HD == 64
  if (T <= 0 || n_items <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, q, pool, block_table, max_pages, positions, row_slot, out, T, H, G, hd, page_tokens, layer,
                    layers_in_group, scale, window);
  if (e) return e;
  if (!item_start) return FELLM_ERR_ARG;
  const int R = H / G;
  const long long rows = n_pages * layers_in_group * 2 * G * page_tokens;
  if (R > PF_WARPS * 16 || page_tokens != DT_PT || window > 0 || rows >= (1ll << 31) || ((uintptr_t)pool & 15)) return FELLM_ERR_SIZE;
  a.item_start = item_start; a.n_items = n_items;
  int tokb = (PF_WARPS * 16) / R; if (tokb < 1) tokb = 1;
  CUtensorMap map;
  e = pool_map_for(pool, rows, DT_PT, &map);
  if (e) return e;
  size_t smem = (size_t)PT_STAGES * 2 * DT_PT * 128 + 1024;
  auto kern = attention_prefill_tma_kernel;
  cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (ce != cudaSuccess) return (int)ce;
  return launch_k_class(launch_class_for_rows(T, 0), kern, dim3((ceil_div(max_item_rows, tokb) + 1) / 2, G, n_items), dim3(PF_WARPS * 32), smem, stream, 1, map, a, status);
#else
  return FELLM_ERR_SIZE;
#endif
}

// Causal attention of prompt portions over the paged cache on the Blackwell tensor path: head size
// 64, pages of 64 tokens, no window.  A CTA takes 128 rows (token, head of one kv head's group) and
// walks over the pages of keys up to its last token:
//   S = Q K^T      tcgen05.mma 128x64x16 (kind::f16), Q and the K page K-major in shared memory
//                  (128-byte swizzle; the page comes by one bulk tensor copy), S in tensor memory;
//   softmax        a row a thread: tcgen05.ld of the row's 64 scores, maximum and sum in registers
//                  with no shuffles, P rounded to bfloat16 into shared memory;
//   O += P V       tcgen05.mma with the V page as the MN-major operand, accumulated in tensor memory.
// The accumulator is scaled by 2^-m with m a row's REFERENCE maximum, which moves only when a tile's
// maximum exceeds it by 2^8: only then is the accumulator read, scaled and written back.
// Two groups of four softmax warps take the even and the odd pages, each with its own reference,
// sum and accumulator, two score tiles (the MMA thread runs two tiles a group ahead) and two P tiles
// (a group need not wait for the MMA that reads the P it has just written); every score tile and P
// tile has barriers of its own, so that no waiter can fall a phase behind.  The groups are merged
// through shared memory at the end.  The exponentials (16 a clock an SM) and the many small MMAs
// bound this kernel; the longest block of a causal prompt sets its duration.
// Roles in a CTA of 320 threads: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) and
// owner of the tensor-memory allocation, warps 2-5 and 6-9 = the softmax groups.
// Every wait on an mbarrier is bounded (a second, or until another role has given up): a role that
// gives up records 311..317 in `status`, and every role falls through to the common exit, where
// tensor memory is freed.
// The same sums as attention_prefill_kernel (attention_mma.cu) up to the order within a row.
//
// FeLLM counterpart: attention_fa2_prefill_paged (plugins/cuda_kernels/src/oxide_kernels.rs:4673,
// one warp per query row).
#include <cuda.h>

#include <mutex>

#include "common.cuh"

#define AU_HD 64
#define AU_PT 64                       // keys per tile: a page
#define AU_ROWS 128
#define AU_STAGES 6                    // pages in flight: the scores run two tiles a group ahead of the softmax
#ifndef AU_GROUPS
#define AU_GROUPS 2                    // softmax groups of four warps; group g takes pages g, g + AU_GROUPS, ...
#endif
#define AU_THREADS (64 + 128 * AU_GROUPS)
#define AU_TILE_B (AU_PT * 128)        // bytes of one K (or V) page tile
#define AU_WAIT_NS 1000000000ull
#define AU_SPIN_LIMIT (1u << 26)

struct AuArgs {
  const bf16* q; const int* block_table; const int* positions; const int* row_slot; const int* item_start;
  bf16* out; int* status;
  int max_pages, H, G, layer, layers_in_group;
  float scale_log2;
};

__device__ __forceinline__ unsigned au_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void au_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void au_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void au_mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool au_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long au_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// Bounded wait: false if the phase has not completed after AU_WAIT_NS (then *status = code and *fail
// is set) or if another role has set *fail meanwhile.
__device__ __forceinline__ bool au_wait(unsigned bar, unsigned parity, volatile int* fail, int* status, int code) {
  if (au_mbar_try(bar, parity)) return true;
  const unsigned long long t0 = au_now();
  for (unsigned i = 0; i < AU_SPIN_LIMIT; ++i) {
    if (au_mbar_try(bar, parity)) return true;
    if ((i & 63) == 63) {
      if (*fail) return false;
      if (au_now() - t0 > AU_WAIT_NS) break;
    }
  }
  *fail = 1;
  if (status) atomicExch(status, code);
  return false;
}
__device__ __forceinline__ void au_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Operand tile with rows of 128 bytes under the 128-byte swizzle, groups of 8 rows 1024 bytes apart:
// K-major (the rows are M or N, the 128 bytes run along K) or MN-major (the rows are K, the 128
// bytes are 64 elements of N); the instruction descriptor says which.
__device__ __forceinline__ unsigned long long au_desc(unsigned smem_addr, bool mn_major = false) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);          // start address
  if (mn_major) d |= (unsigned long long)(8192 >> 4) << 16;       // leading byte offset: the next 64 elements of MN (there are none here)
  d |= (unsigned long long)(1024 >> 4) << 32;                     // stride byte offset: the next group of 8 rows
  d |= 1ull << 46;                                                // descriptor version (sm_100)
  d |= 2ull << 61;                                                // SWIZZLE_128B
  return d;
}
// kind::f16: D float32, A and B bfloat16; b_mn: B is MN-major (bit 16); N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ unsigned au_idesc(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void au_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void au_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void au_tmem_ld32_issue(unsigned taddr, float* v) {
  unsigned* r = reinterpret_cast<unsigned*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void au_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void au_tmem_ld32(unsigned taddr, float* v) {
  au_tmem_ld32_issue(taddr, v);
  au_tmem_ld_wait();
}
__device__ __forceinline__ void au_tmem_st32(unsigned taddr, const float* v) {
  const unsigned* r = reinterpret_cast<const unsigned*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
         "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
         "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
         "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void au_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void au_st_shared16(unsigned addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// byte offset of 16-byte chunk `chunk` of row `row` in a tile of 128-byte rows under the 128-byte swizzle
__device__ __forceinline__ unsigned au_off(int row, int chunk) { return (unsigned)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ float au_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Tensor memory columns: two score tiles (one being read while the MMA thread fills the other) and an
// accumulator of P V for each softmax group.
#define AU_COL_S 0
#define AU_COL_O (2 * AU_GROUPS * AU_PT)
#define AU_TMEM_COLS 512
static_assert(3 * AU_GROUPS * 64 <= AU_TMEM_COLS, "tensor memory: 192 columns a group");
#define AU_MERGE_STRIDE (AU_HD + 2)    // floats of a row's record in the merge buffer: o, m, l
#define AU_RESCALE_AT 8.0f             // a row's reference maximum moves when a tile's maximum is 2^8 above it

__global__ void __launch_bounds__(AU_THREADS, 1)
attention_prefill_umma_kernel(const __grid_constant__ CUtensorMap pool_map, AuArgs a) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_PREFILL);
  extern __shared__ unsigned char smem_raw[];
  // full[STAGES], empty[STAGES], q_ready, s_full[GROUPS][2], p_full[GROUPS][2], o_full[GROUPS][2]: a barrier
  // for each of a group's two score tiles and two P tiles, so that no waiter is ever a phase behind
  __shared__ __align__(8) unsigned long long bars[2 * AU_STAGES + 1 + 6 * AU_GROUPS];
  __shared__ unsigned tmem_base_s;
  __shared__ int sm_fail;
  const int item = blockIdx.z;
  const int g = blockIdx.x % a.G, rank = blockIdx.x / a.G;     // CTAs in launch order: the longest blocks of every kv head first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = a.H / a.G;                                     // divides 128 (the launcher checks)
  const int tokb = AU_ROWS / R;                                // tokens a CTA
  pdl_launch_dependents();
  const int row_begin = a.item_start[item], n_rows = a.item_start[item + 1] - row_begin;
  const int n_blocks = (n_rows + tokb - 1) / tokb;
  if (rank >= n_blocks) return;                                // before any barrier or allocation
  const int blk = n_blocks - 1 - rank;
  const int tok0 = blk * tokb, n_tok = min(tokb, n_rows - tok0);
  const int pos0 = a.positions[row_begin] + tok0;              // position of the block's first token
  const int k_last = pos0 + n_tok - 1;
  const int n_tiles = k_last / AU_PT + 1;                      // pages 0 .. that of the last token
  const int* bt = a.block_table + (size_t)a.row_slot[row_begin] * a.max_pages;

  const unsigned base = (au_smem(smem_raw) + 1023u) & ~1023u;  // the swizzle is by address
  unsigned char* base_ptr = smem_raw + (base - au_smem(smem_raw));
  const unsigned q_s = base, p_s0 = base + AU_ROWS * 128, stage0 = base + (1 + 2 * AU_GROUPS) * AU_ROWS * 128;
  float* merge = (float*)(base_ptr + AU_ROWS * 128);           // over the P tiles and the stages, once every MMA is done
  const unsigned full0 = au_smem(&bars[0]), empty0 = au_smem(&bars[AU_STAGES]);
  const unsigned q_ready = au_smem(&bars[2 * AU_STAGES]), s_full0 = q_ready + 8, p_full0 = s_full0 + 16 * AU_GROUPS,
                 o_full0 = p_full0 + 16 * AU_GROUPS;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AU_STAGES; ++s) { au_mbar_init(full0 + 8 * s, 1); au_mbar_init(empty0 + 8 * s, 1); }
    au_mbar_init(q_ready, 4);
    for (int b = 0; b < AU_GROUPS; ++b) {
      au_mbar_init(s_full0 + 16 * b, 1); au_mbar_init(s_full0 + 16 * b + 8, 1); au_mbar_init(p_full0 + 16 * b, 4); au_mbar_init(p_full0 + 16 * b + 8, 4);
      au_mbar_init(o_full0 + 16 * b, 1); au_mbar_init(o_full0 + 16 * b + 8, 1);
    }
    sm_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(au_smem(&tmem_base_s)), "r"(AU_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  volatile int* fail = &sm_fail;
  pdl_wait(); FELLM_TRACE_WAITED();                            // q and the cache rows of this step come from the kernel before

  if (warp == 0) {
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % AU_STAGES;
        if (j >= AU_STAGES && !au_wait(empty0 + 8 * s, (j / AU_STAGES - 1) & 1, fail, a.status, 311)) break;
        const int page = max(bt[j], 0);                        // an unmapped entry (-1) must never become an address
        const int row = (((page * a.layers_in_group + a.layer) * 2) * a.G + g) * AU_PT;      // < 2^31: the launcher checks
        const unsigned dst = stage0 + s * 2 * AU_TILE_B;
        au_mbar_expect_tx(full0 + 8 * s, 2 * AU_TILE_B);
        au_tma_load_2d(dst, &pool_map, 0, row, full0 + 8 * s);
        au_tma_load_2d(dst + AU_TILE_B, &pool_map, 0, row + a.G * AU_PT, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // tile j belongs to softmax group j % GROUPS: its score tile, P tile, accumulator and barriers
      const unsigned idesc_s = au_idesc(AU_ROWS, AU_PT, false), idesc_o = au_idesc(AU_ROWS, AU_HD, true);
      const unsigned long long dq = au_desc(q_s);
      auto scores = [&](int j) -> bool {                       // S_j = Q K_j^T into the group's score tile (j / GROUPS) & 1
        const int s = j % AU_STAGES, grp = j % AU_GROUPS, sb = (j / AU_GROUPS) & 1;
        if (!au_wait(full0 + 8 * s, (j / AU_STAGES) & 1, fail, a.status, 312)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned long long dk = au_desc(stage0 + s * 2 * AU_TILE_B);
#pragma unroll
        for (int k = 0; k < AU_HD / 16; ++k)                   // 32 bytes further along the head inside the swizzle atom
          au_mma(tmem_base + AU_COL_S + (2 * grp + sb) * AU_PT, dq + (unsigned long long)(k * 2), dk + (unsigned long long)(k * 2), idesc_s, k ? 1u : 0u);
        au_commit(s_full0 + 16 * grp + 8 * sb);
        return true;
      };
      bool ok = au_wait(q_ready, 0, fail, a.status, 313);
      if (ok) asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      for (int j = 0; j < 2 * AU_GROUPS && j < n_tiles && ok; ++j) ok = scores(j);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % AU_STAGES, grp = j % AU_GROUPS, i = j / AU_GROUPS;
        // P_j lies in shared memory, S_j has been read, and the accumulator is scaled to P_j's reference
        ok = au_wait(p_full0 + 16 * grp + 8 * (i & 1), (i >> 1) & 1, fail, a.status, 314);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned long long dp = au_desc(p_s0 + (2 * grp + (i & 1)) * AU_ROWS * 128);
        const unsigned long long dv = au_desc(stage0 + s * 2 * AU_TILE_B + AU_TILE_B, true);
#pragma unroll
        for (int k = 0; k < AU_PT / 16; ++k)                   // 16 keys further: 32 bytes along P's rows, 16 rows (2048 bytes) down V
          au_mma(tmem_base + AU_COL_O + grp * AU_HD, dp + (unsigned long long)(k * 2), dv + (unsigned long long)(k * 128), idesc_o,
                 (i | k) ? 1u : 0u);                           // the group's first tile starts its accumulator
        au_commit(o_full0 + 16 * grp + 8 * (i & 1));
        au_commit(empty0 + 8 * s);                             // the page's stage is free once these MMAs have read it
        if (j + 2 * AU_GROUPS < n_tiles) ok = scores(j + 2 * AU_GROUPS);   // into the score tile that S_j has left
      }
    }
  } else {
    // softmax warps: TMEM lanes 32*(warp%4) .. +32 = the CTA's rows, a row a thread; group = which pages
    const int grp = (warp - 2) >> 2, qd = warp & 3, row = qd * 32 + lane;
    const int tok = row / R, head = row - tok * R;
    const bool valid = tok < n_tok;
    const int pos = pos0 + tok;
    const size_t out_row = ((size_t)(row_begin + tok0 + tok) * a.H + g * R + head) * AU_HD;
    if (grp == 0) {
      const uint4* src = (const uint4*)(a.q + out_row);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) au_st_shared16(q_s + au_off(row, ch), valid ? src[ch] : make_uint4(0, 0, 0, 0));
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // these writes before the MMA's reads
      __syncwarp();
      if (lane == 0) au_mbar_arrive(q_ready);
    }
    const unsigned t_row = tmem_base + ((unsigned)(qd * 32) << 16);
    const unsigned t_acc = t_row + AU_COL_O + grp * AU_HD;
    const unsigned s_full = s_full0 + 16 * grp, p_full = p_full0 + 16 * grp, o_full = o_full0 + 16 * grp;
    const float scale = a.scale_log2;
    // The accumulator of P V stays in tensor memory, scaled by 2^-m where m is the row's REFERENCE
    // maximum; m only moves when a tile's maximum exceeds it by AU_RESCALE_AT (P then stays below 2^8,
    // well inside bfloat16 and float32), and only then is the accumulator read, scaled and written back.
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    int n_mine = 0;
    for (int j = grp; j < n_tiles; j += AU_GROUPS, ++n_mine) {
      const int key0 = j * AU_PT, s = j % AU_STAGES, i = n_mine;
      if (key0 + AU_PT > k_last + 1) {
        // rows past the last key hold whatever the page held before: zero the V rows, so that 0 * V is 0
        ok = au_wait(full0 + 8 * s, (j / AU_STAGES) & 1, fail, a.status, 315);
        if (!ok) break;
        const unsigned v_s = stage0 + s * 2 * AU_TILE_B + AU_TILE_B;
        for (int e = (k_last + 1 - key0) * 8 + row; e < AU_PT * 8; e += AU_ROWS)
          au_st_shared16(v_s + au_off(e >> 3, e & 7), make_uint4(0, 0, 0, 0));
      }
      ok = au_wait(s_full + 8 * (i & 1), (i >> 1) & 1, fail, a.status, 316);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      float sc[AU_PT];
      au_tmem_ld32_issue(t_row + AU_COL_S + (2 * grp + (i & 1)) * AU_PT, sc);
      au_tmem_ld32_issue(t_row + AU_COL_S + (2 * grp + (i & 1)) * AU_PT + 32, sc + 32);
      au_tmem_ld_wait();
      if (key0 + AU_PT - 1 > pos) {
#pragma unroll
        for (int c = 0; c < AU_PT; ++c) sc[c] = (key0 + c <= pos) ? sc[c] : -INFINITY;
      }
      float r4[4] = {sc[0], sc[1], sc[2], sc[3]};               // four chains, not one of 63 dependent steps
#pragma unroll
      for (int c = 4; c < AU_PT; c += 4) {
        r4[0] = fmaxf(r4[0], sc[c]); r4[1] = fmaxf(r4[1], sc[c + 1]); r4[2] = fmaxf(r4[2], sc[c + 2]); r4[3] = fmaxf(r4[3], sc[c + 3]);
      }
      const float tile_max = fmaxf(fmaxf(r4[0], r4[1]), fmaxf(r4[2], r4[3])) * scale;      // the scale is positive
      // A tile may hold no key that a row sees (a later group's first page lies behind the rows of a
      // block's first positions): its maximum is -inf, nothing moves and P is zero.
      const bool move = tile_max > m + AU_RESCALE_AT || (m == -INFINITY && tile_max > -INFINITY);
      float corr = 1.f;
      if (move) {
        corr = (m == -INFINITY) ? 0.f : au_ex2(m - tile_max);
        m = tile_max;
        l *= corr;
      }
      const bool none = m == -INFINITY;
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned pk[AU_PT / 2];
#pragma unroll
      for (int c = 0; c < AU_PT; c += 4) {
        float p0 = au_ex2(fmaf(sc[c], scale, -m)), p1 = au_ex2(fmaf(sc[c + 1], scale, -m));
        float p2 = au_ex2(fmaf(sc[c + 2], scale, -m)), p3 = au_ex2(fmaf(sc[c + 3], scale, -m));
        if (none) { p0 = p1 = p2 = p3 = 0.f; }                  // -inf - -inf is not a number
        s4[0] += p0; s4[1] += p1; s4[2] += p2; s4[3] += p3;
        __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
        pk[c >> 1] = *(unsigned*)&pa; pk[(c >> 1) + 1] = *(unsigned*)&pb;
      }
      l += (s4[0] + s4[1]) + (s4[2] + s4[3]);
      // two P tiles a group: this one is free once the MMA of the group's tile before the last has read it
      if (i > 1) {
        ok = au_wait(o_full + 8 * (i & 1), ((i - 2) >> 1) & 1, fail, a.status, 317);
        if (!ok) break;
      }
      if (i > 0 && __any_sync(0xffffffffu, move)) {
        // some row of the warp moved its reference: scale the warp's rows of the accumulator, once the
        // MMA of the tile before has added into it
        ok = au_wait(o_full + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, fail, a.status, 317);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          float ot[32];
          au_tmem_ld32(t_acc + 32 * hlf, ot);
#pragma unroll
          for (int d = 0; d < 32; ++d) ot[d] *= corr;
          au_tmem_st32(t_acc + 32 * hlf, ot);
        }
        au_tmem_st_wait();
      }
      const unsigned p_s = p_s0 + (2 * grp + (i & 1)) * AU_ROWS * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        au_st_shared16(p_s + au_off(row, ch), make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]));
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // P (and the zeroed V rows) before the MMA's reads
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) au_mbar_arrive(p_full + 8 * (i & 1));
    }
    float o[AU_HD];
    if (ok && n_mine > 0) {
      ok = au_wait(o_full + 8 * ((n_mine - 1) & 1), ((n_mine - 1) >> 1) & 1, fail, a.status, 317);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        au_tmem_ld32_issue(t_acc, o);
        au_tmem_ld32_issue(t_acc + 32, o + 32);
        au_tmem_ld_wait();
      }
    }
    if (n_mine == 0 || !ok) {
#pragma unroll
      for (int d = 0; d < AU_HD; ++d) o[d] = 0.f;
    }
    // Every group is through its last tile: every MMA and every copy of this CTA is done, and the P
    // tiles and stages are free for the later groups' records.  (A group that gave up still comes to
    // the barriers; the result is then not stored.)
    asm volatile("bar.sync 1, %0;\n" ::"n"(128 * AU_GROUPS) : "memory");
    if (grp > 0) {
      float* rec = merge + ((size_t)(grp - 1) * AU_ROWS + row) * AU_MERGE_STRIDE;
#pragma unroll
      for (int d = 0; d < AU_HD; ++d) rec[d] = o[d];
      rec[AU_HD] = m; rec[AU_HD + 1] = l;
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(128 * AU_GROUPS) : "memory");
    if (grp == 0 && ok && !*fail && valid) {
      float mm = m;                                            // group 0 has page 0: m is finite
#pragma unroll
      for (int q = 0; q < AU_GROUPS - 1; ++q) mm = fmaxf(mm, merge[((size_t)q * AU_ROWS + row) * AU_MERGE_STRIDE + AU_HD]);
      const float c0 = au_ex2(m - mm);
      float lt = l * c0;
#pragma unroll
      for (int d = 0; d < AU_HD; ++d) o[d] *= c0;
#pragma unroll
      for (int q = 0; q < AU_GROUPS - 1; ++q) {
        const float* rec = merge + ((size_t)q * AU_ROWS + row) * AU_MERGE_STRIDE;
        const float mq = rec[AU_HD], cq = (mq == -INFINITY) ? 0.f : au_ex2(mq - mm);
        lt = fmaf(rec[AU_HD + 1], cq, lt);
#pragma unroll
        for (int d = 0; d < AU_HD; ++d) o[d] = fmaf(rec[d], cq, o[d]);
      }
      const float inv = 1.0f / lt;
      uint4* dst = (uint4*)(a.out + out_row);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        __nv_bfloat162 q0 = __floats2bfloat162_rn(o[8 * ch] * inv, o[8 * ch + 1] * inv), q1 = __floats2bfloat162_rn(o[8 * ch + 2] * inv, o[8 * ch + 3] * inv);
        __nv_bfloat162 q2 = __floats2bfloat162_rn(o[8 * ch + 4] * inv, o[8 * ch + 5] * inv), q3 = __floats2bfloat162_rn(o[8 * ch + 6] * inv, o[8 * ch + 7] * inv);
        dst[ch] = make_uint4(*(unsigned*)&q0, *(unsigned*)&q1, *(unsigned*)&q2, *(unsigned*)&q3);
      }
    }
  }
  // common exit: every role comes here, also after a wait that gave up
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(AU_TMEM_COLS) : "memory");
  }
}

// The cache pool as a 2-D tensor [rows of 64 dims], a page of one kv head (64 rows) a box: the map is
// kept per (pool, rows).
typedef CUresult (*AuEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int au_pool_map(const void* pool, long long rows, CUtensorMap* out) {
  static std::mutex mu;
  static struct { const void* pool; long long rows; CUtensorMap map; } cache[8];
  static int n_cached = 0, next = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_cached; ++i)
    if (cache[i].pool == pool && cache[i].rows == rows) { *out = cache[i].map; return 0; }
  static AuEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return FELLM_ERR_ARG;
    fn = (AuEncodeTiledFn)p;
  }
  cuuint64_t dims[2] = {(cuuint64_t)AU_HD, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)AU_HD * 2};
  cuuint32_t box[2] = {AU_HD, AU_PT};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  cache[next].pool = pool; cache[next].rows = rows; cache[next].map = m;
  next = (next + 1) % 8;
  if (n_cached < 8) ++n_cached;
  *out = m;
  return 0;
}

// Whether fellm_attn_prefill_umma takes these sizes (1) or not (0).
FELLM_API int fellm_attn_prefill_umma_takes(int H, int G, int hd, int page_tokens, int window) {
  if (G < 1 || H % G) return 0;
  const int R = H / G;
  return (hd == AU_HD && page_tokens == AU_PT && window <= 0 && R <= AU_ROWS && AU_ROWS % R == 0) ? 1 : 0;
}

// q [T, H, 64] bfloat16 (normed, rotated), out [T, H*64]; pool [n_pages, layers_in_group, 2, G, 64, 64];
// rows of item i are item_start[i]..item_start[i+1], its positions are consecutive from
// positions[item_start[i]]; max_item_rows: the longest item of the step.  status: device int32 that a
// role sets (311..317) if a wait ran out.  FELLM_ERR_SIZE for sizes it does not take.
FELLM_API int fellm_attn_prefill_umma(const void* q, const void* pool, long long n_pages, const int* block_table,
                                      int max_pages, const int* positions, const int* row_slot, const int* item_start,
                                      int n_items, int max_item_rows, void* out, int T, int H, int G, int hd,
                                      int page_tokens, int layer, int layers_in_group, float scale, int window,
                                      int* status, cudaStream_t stream) {
  if (T <= 0 || n_items <= 0) return 0;
  if (!q || !pool || !block_table || !positions || !row_slot || !item_start || !out) return FELLM_ERR_ARG;
  if (!fellm_attn_prefill_umma_takes(H, G, hd, page_tokens, window)) return FELLM_ERR_SIZE;
  const long long rows = n_pages * layers_in_group * 2 * G * page_tokens;
  if (rows >= (1ll << 31) || ((uintptr_t)pool & 15) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return FELLM_ERR_SIZE;
  AuArgs a;
  a.q = (const bf16*)q; a.block_table = block_table; a.positions = positions; a.row_slot = row_slot; a.item_start = item_start;
  a.out = (bf16*)out; a.status = status; a.max_pages = max_pages; a.H = H; a.G = G; a.layer = layer;
  a.layers_in_group = layers_in_group; a.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap map;
  int e = au_pool_map(pool, rows, &map);
  if (e) return e;
  const int tokb = AU_ROWS / (H / G);
  size_t smem = (size_t)(1 + 2 * AU_GROUPS) * AU_ROWS * 128 + (size_t)AU_STAGES * 2 * AU_TILE_B + 1024;     // Q, the P tiles, the stages
  auto kern = attention_prefill_umma_kernel;
  cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (ce != cudaSuccess) return (int)ce;
  return launch_k_class(launch_class_for_rows(T, 0), kern, dim3(ceil_div(max_item_rows, tokb) * G, 1, n_items), dim3(AU_THREADS), smem, stream, 1, map, a);
}

// C[M,N] = A[M,K] W[N,K]^T for many rows (prefill), bfloat16 operands, float32 accumulation in
// tensor memory: the Blackwell path.  tcgen05.mma (cta_group::1, kind::f16, 128x128x16) issued by
// one thread, operands brought by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a ring of
// five 32 KB stages, accumulator read back with tcgen05.ld for a fused epilogue: store, add into
// the float32 residual stream, SiLU(gate)*up over weight rows interleaved in blocks of 8, float32
// store.
//
// Roles in a CTA of 320 threads: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane)
// and owner of the tensor-memory allocation, warps 2-9 = epilogue (TMEM lane quarter = warp % 4,
// column half = (warp - 2) / 4).
// Every wait on an mbarrier is bounded: after a second of polling a role records the barrier it gave up
// on in `status`, and all roles fall through to the common exit, where tensor memory is freed.
//
// FeLLM counterpart: bf16_matmul_rows, one thread per output
// (plugins/cuda_kernels/src/oxide_kernels.rs:3165).
#include <cuda.h>
#include <cooperative_groups.h>
namespace cgx = cooperative_groups;

#define FELLM_WEIGHT_PREFETCH 1
#include "common.cuh"

#define UM_BM 128
#define UM_BK 64                      // one 128-byte swizzle atom of bfloat16 per row
#define UM_STAGES 5                   // 160 KB of stages in flight ahead of the MMA thread; one persistent CTA per SM
#define UM_THREADS 320                // TMA warp, MMA warp, 8 epilogue warps
#define UM_SPIN_LIMIT (1u << 26)
#define UM_WAIT_NS 1000000000ull       // one second: far beyond any healthy wait, short enough to stay responsive

enum { EPI_STORE = 0, EPI_ACC = 1, EPI_SWIGLU = 2, EPI_F32 = 3, EPI_CONV = 4 };      // 4: only the product of few rows

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// Bounded wait: false (and *status set) if the phase has not completed after UM_WAIT_NS.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (unsigned i = 0; i < UM_SPIN_LIMIT; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 63) == 63 && global_ns() - t0 > UM_WAIT_NS) break;
  }
  if (status) atomicExch(status, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major operand tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);          // start address
  d |= (unsigned long long)(1024 >> 4) << 32;                     // stride byte offset: next 8-row group
  d |= 1ull << 46;                                                // descriptor version (sm_100)
  d |= 2ull << 61;                                                // SWIZZLE_128B
  return d;
}
// kind::f16: D float32, A and B bfloat16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ unsigned umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                         unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float* v) {
  unsigned* r = reinterpret_cast<unsigned*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

struct UmmaArgs {
  const float* bias; void* out; int* status;
  int M, N, K, ldo;
};

// One 32-column chunk of an output row: v[j] is C[m][n + j].
// `res`: for EPI_ACC, the 32 values out already holds there, loaded while the MMAs ran (or null).
template <int EPI>
__device__ __forceinline__ void store_chunk(const UmmaArgs& a, float* v, int m, int n, const float4* res = nullptr) {
  if (EPI == EPI_SWIGLU) {
    // columns: 8 gate, 8 up, 8 gate, 8 up -> 16 features
    bf16* dst = (bf16*)a.out + (size_t)m * a.ldo + (n >> 1);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (n + 16 * h >= a.N) break;
      unsigned packed[4];
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        float g0 = v[16 * h + j], g1 = v[16 * h + j + 1], u0 = v[16 * h + 8 + j], u1 = v[16 * h + 9 + j];
        if (a.bias) { g0 += a.bias[n + 16 * h + j]; g1 += a.bias[n + 16 * h + j + 1]; u0 += a.bias[n + 16 * h + 8 + j]; u1 += a.bias[n + 16 * h + 9 + j]; }
        __nv_bfloat162 p = __floats2bfloat162_rn((g0 / (1.0f + expf(-g0))) * u0, (g1 / (1.0f + expf(-g1))) * u1);
        packed[j >> 1] = *(unsigned*)&p;
      }
      *(uint4*)(dst + 8 * h) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    return;
  }
  const bool whole = n + 32 <= a.N;
  if (a.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j) if (n + j < a.N) v[j] += a.bias[n + j];
  }
  if (EPI == EPI_STORE && whole && (a.ldo % 8) == 0) {
    uint4* dst = (uint4*)((bf16*)a.out + (size_t)m * a.ldo + n);         // 64 contiguous bytes of this row
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]), p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]), p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
      dst[j] = make_uint4(*(unsigned*)&p0, *(unsigned*)&p1, *(unsigned*)&p2, *(unsigned*)&p3);
    }
  } else if (EPI != EPI_STORE && whole && (a.ldo % 4) == 0) {
    float4* dst = (float4*)((float*)a.out + (size_t)m * a.ldo + n);       // 128 contiguous bytes of this row
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 r = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      if (EPI == EPI_ACC) { float4 o = res ? res[j] : dst[j]; r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w; }
      dst[j] = r;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (n + j >= a.N) break;
      size_t o = (size_t)m * a.ldo + n + j;
      if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(v[j]);
      else if (EPI == EPI_ACC) ((float*)a.out)[o] += v[j];
      else ((float*)a.out)[o] = v[j];
    }
  }
}

// Persistent: a CTA walks over output tiles t = blockIdx.x, + gridDim.x, ... (tiles that follow one another share
// their weight tile).  Two accumulators in tensor memory: while the epilogue warps read tile i out of one, the MMA
// thread fills the other with tile i+1, and the TMA thread is already fetching operands further ahead.
template <int EPI, int BN>
__global__ void __launch_bounds__(UM_THREADS)
gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, UmmaArgs a) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_UMMA);
  constexpr int STAGES = BN == 256 ? 4 : UM_STAGES;         // 48 KB or 32 KB a stage
  constexpr int STAGE_BYTES = (UM_BM + BN) * UM_BK * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * STAGES + 4];    // full[], empty[], acc_full[2], acc_empty[2]
  __shared__ unsigned tmem_base_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the dynamic buffer is aligned by hand: swizzled TMA tiles want 1024 bytes
  unsigned tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const unsigned full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const unsigned accfull0 = smem_u32(&bars[2 * STAGES]), accempty0 = smem_u32(&bars[2 * STAGES + 2]);
  const int k_blocks = (a.K + UM_BK - 1) / UM_BK;
  const int m_tiles = (a.M + UM_BM - 1) / UM_BM, n_tiles = (a.N + BN - 1) / BN, total = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accfull0 + 8 * b, 1); mbar_init(accempty0 + 8 * b, 8); }   // 8 epilogue warps
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {                   // tensor memory: two 128x128 float32 accumulators = 256 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();                        // A is the output of the kernel before this one

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;               // k-blocks issued so far, over all tiles: stage = it % STAGES
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * UM_BM, n0 = (t / m_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(empty0 + 8 * s, (it / STAGES - 1) & 1, a.status, 101)) { ok = false; break; }
          unsigned dst = tiles + s * STAGE_BYTES;
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          tma_load_2d(dst, &map_a, kb * UM_BK, m0, full0 + 8 * s);
          tma_load_2d(dst + UM_BM * UM_BK * 2, &map_w, kb * UM_BK, n0, full0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = umma_idesc(UM_BM, BN);
      unsigned it = 0, use = 0;      // use: tiles done so far; accumulator = use & 1
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++use) {
        const unsigned acc = use & 1, d_tmem = tmem_base + acc * BN;
        if (use >= 2) {              // the epilogue must have drained this accumulator's previous tile
          ok = mbar_wait(accempty0 + 8 * acc, ((use >> 1) - 1) & 1, a.status, 104);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, a.status, 102);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          unsigned sa = tiles + s * STAGE_BYTES, sb = sa + UM_BM * UM_BK * 2;
          unsigned long long da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
          for (int k = 0; k < UM_BK / 16; ++k)          // 32 bytes further along K inside the swizzle atom
            umma_f16(d_tmem, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);                  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(accfull0 + 8 * acc);        // arrives when every MMA of this tile is done
      }
    }
  } else {
    // epilogue warps: TMEM lanes 32*(warp%4) .. +32 = output rows; two warps share a quarter, a column half each
    const int q = warp & 3, half = (warp - 2) >> 2;
    unsigned use = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++use) {
      const unsigned acc = use & 1;
      const int m0 = (t % m_tiles) * UM_BM, n0 = (t / m_tiles) * BN;
      const int m = m0 + q * 32 + lane;
      // += residual: what out holds in this thread's two chunks is fetched while the MMAs of the
      // tile still run (nothing else writes these elements during the launch)
      constexpr int CHUNKS = BN / 2 / 32;
      constexpr int PRE = CHUNKS < 2 ? CHUNKS : 2;               // chunks fetched ahead (64 registers)
      float4 res[EPI == EPI_ACC ? PRE : 1][8];
      bool res_ok[CHUNKS];
#pragma unroll
      for (int ch = 0; ch < CHUNKS; ++ch) {
        const int n = n0 + half * (BN / 2) + ch * 32;
        res_ok[ch] = EPI == EPI_ACC && ch < PRE && m < a.M && n + 32 <= a.N && (a.ldo % 4) == 0;
        if (EPI == EPI_ACC && res_ok[ch]) {
          const float4* src = (const float4*)((const float*)a.out + (size_t)m * a.ldo + n);
#pragma unroll
          for (int j = 0; j < 8; ++j) res[ch][j] = src[j];
        }
      }
      if (!mbar_wait(accfull0 + 8 * acc, (use >> 1) & 1, a.status, 103)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
      for (int ch = 0; ch < CHUNKS; ++ch) {
        const int c0 = half * (BN / 2) + ch * 32;
        float v[32];
        tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + acc * BN + (unsigned)c0, v);      // whole warp, also for rows past M
        if (m < a.M && n0 + c0 < a.N) store_chunk<EPI>(a, v, m, n0 + c0, (EPI == EPI_ACC && res_ok[ch]) ? res[ch < PRE ? ch : 0] : nullptr);
      }
      // this warp has read its part of the accumulator: one of the eight arrivals that free it
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(accempty0 + 8 * acc) : "memory");
    }
  }
  // common exit: every role comes here, also after a wait that gave up
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// K over a cluster of two: a product of a few hundred rows (prompt portions beside decode tokens) with a narrow N
// has few 128 x 128 tiles for 148 SMs and a long K for each of them.  Here every tile is the work of TWO CTAs, each
// with half of the k-blocks (own TMA, own MMAs, own tensor memory, as in the kernel above); the second CTA's epilogue
// warps send their float32 partial tile to the first CTA's shared memory (st.shared::cluster, rows 528 bytes apart),
// arrive on a barrier there, and the first CTA's epilogue adds the two parts (own first, then the other's: a fixed
// order) and runs the epilogue.  One tile a cluster, no tile loop.  Waits bounded: status 131 producer, 132 MMA,
// 133 accumulator, 134 the other CTA's part.
#define UK_STAGES 4
#define UK_RECV_LD (UM_BM + 4)        // floats between rows of the received tile
__device__ __forceinline__ unsigned cluster_ctarank();
__device__ __forceinline__ unsigned mapa_u32(unsigned smem_addr, unsigned rank);
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr);
__device__ __forceinline__ bool mbar_wait_cluster(unsigned bar, unsigned parity, int* status, int code) {
  // (the phase was completed by arrivals of another CTA: acquire at cluster scope, so that what it stored before is seen)
  const unsigned long long t0 = global_ns();
  for (unsigned i = 0; i < UM_SPIN_LIMIT; ++i) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 63) == 63 && global_ns() - t0 > UM_WAIT_NS) break;
  }
  if (status) atomicExch(status, code);
  return false;
}
__device__ __forceinline__ void st_cluster_v4(unsigned addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(UM_THREADS)
gemm_umma_ksplit_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, UmmaArgs a) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_UMMA);
  constexpr int BN = 128, STAGE_BYTES = (UM_BM + BN) * UM_BK * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * UK_STAGES + 2];    // full[], empty[], accumulator done, the other's part here
  __shared__ unsigned tmem_base_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  float* recv = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + (size_t)UK_STAGES * STAGE_BYTES);
  const unsigned full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[UK_STAGES]);
  const unsigned accfull = smem_u32(&bars[2 * UK_STAGES]), recvfull = smem_u32(&bars[2 * UK_STAGES + 1]);
  const unsigned rank = cluster_ctarank();
  const int k_blocks = (a.K + UM_BK - 1) / UM_BK;
  const int kb_lo = rank == 0 ? 0 : k_blocks / 2, kb_hi = rank == 0 ? k_blocks / 2 : k_blocks;     // (k_blocks >= 2: the launcher checks)
  const int m_tiles = (a.M + UM_BM - 1) / UM_BM;
  const int t = blockIdx.x >> 1;
  const int m0 = (t % m_tiles) * UM_BM, n0 = (t / m_tiles) * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < UK_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(accfull, 1);
    mbar_init(recvfull, 8);                                  // the other CTA's eight epilogue warps
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  cgx::this_cluster().sync();                                // both CTAs run and their barriers are set up
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();                        // A is the output of the kernel before this one

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = kb_lo, it = 0; kb < kb_hi; ++kb, ++it) {
        const int s = it % UK_STAGES;
        if (it >= UK_STAGES && !mbar_wait(empty0 + 8 * s, (it / UK_STAGES - 1) & 1, a.status, 131)) break;
        const unsigned dst = tiles + s * STAGE_BYTES;
        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        tma_load_2d(dst, &map_a, kb * UM_BK, m0, full0 + 8 * s);
        tma_load_2d(dst + UM_BM * UM_BK * 2, &map_w, kb * UM_BK, n0, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = umma_idesc(UM_BM, BN);
      bool ok = true;
      for (int kb = kb_lo, it = 0; kb < kb_hi; ++kb, ++it) {
        const int s = it % UK_STAGES;
        ok = mbar_wait(full0 + 8 * s, (it / UK_STAGES) & 1, a.status, 132);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned sa = tiles + s * STAGE_BYTES, sb = sa + UM_BM * UM_BK * 2;
        const unsigned long long da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
        for (int k = 0; k < UM_BK / 16; ++k)
          umma_f16(tmem_base, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc, (it | k) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);
      }
      if (ok) umma_commit(accfull);
    }
  } else {
    // epilogue warps: TMEM lanes 32*(warp%4) .. +32 = output rows; two warps share a quarter, a column half each
    const int q = warp & 3, half = (warp - 2) >> 2, row = q * 32 + lane;
    const int m = m0 + row;
    constexpr int CHUNKS = BN / 2 / 32;                       // 2
    float4 res[EPI == EPI_ACC ? CHUNKS : 1][8];
    bool res_ok[CHUNKS];
#pragma unroll
    for (int ch = 0; ch < CHUNKS; ++ch) {
      const int n = n0 + half * (BN / 2) + ch * 32;
      res_ok[ch] = EPI == EPI_ACC && rank == 0 && m < a.M && n + 32 <= a.N && (a.ldo % 4) == 0;
      if (EPI == EPI_ACC && res_ok[ch]) {
        const float4* src = (const float4*)((const float*)a.out + (size_t)m * a.ldo + n);
#pragma unroll
        for (int j = 0; j < 8; ++j) res[ch][j] = src[j];
      }
    }
    const bool done = mbar_wait(accfull, 0, a.status, 133);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (rank == 1) {
      // this CTA's part goes to the first CTA, row by row as the tensor memory gives it
      const unsigned there = mapa_u32(smem_u32(recv), 0);
      if (done) {
#pragma unroll
        for (int ch = 0; ch < CHUNKS; ++ch) {
          const int c0 = half * (BN / 2) + ch * 32;
          float v[32];
          tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)c0, v);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_cluster_v4(there + (unsigned)((row * UK_RECV_LD + c0 + 4 * j) * 4), make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(recvfull, 0));       // (release at cluster scope: the stores above come first)
    } else {
      const bool got = mbar_wait_cluster(recvfull, 0, a.status, 134);
      if (done && got) {
#pragma unroll
        for (int ch = 0; ch < CHUNKS; ++ch) {
          const int c0 = half * (BN / 2) + ch * 32;
          float v[32];
          tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)c0, v);
          const float4* other = reinterpret_cast<const float4*>(recv + row * UK_RECV_LD + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 o = other[j];
            v[4 * j] += o.x; v[4 * j + 1] += o.y; v[4 * j + 2] += o.z; v[4 * j + 3] += o.w;
          }
          if (m < a.M && n0 + c0 < a.N) store_chunk<EPI>(a, v, m, n0 + c0, (EPI == EPI_ACC && res_ok[ch]) ? res[ch] : nullptr);
        }
      }
    }
  }
  // common exit: every role comes here, also after a wait that gave up.  The second CTA may leave before the first
  // (nobody reads its shared memory); the first leaves after it has taken the other's part, or given up on it.
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(BN) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster, on the two SMs of a TPC, work on ONE tile
// of 256 rows x BN columns.  Each CTA brings its own 128 rows of A and HALF of the tile's W rows
// (BN / 2) by TMA into its own shared memory; the MMA, issued by one thread of the pair's first
// CTA, reads both CTAs' shared memory and writes each CTA's 128 rows of the accumulator into that
// CTA's tensor memory.  A 256 x 256 tile then costs a CTA 32 KB of operands a k-block where the
// single-CTA 128 x 256 tile costs 48 KB and the 128 x 128 tile 32 KB for a quarter of the product:
// the kernel above is bound by operand bytes from L2, this one moves half as many a FLOP.
// No multicast load anywhere: both CTAs fetch their own halves.
//
// What the pair shares, as the PTX ISA gives it (cta_group::2 forms of tcgen05.alloc / mma / commit,
// cp.async.bulk.tensor with .cta_group::2 completing bytes on the first CTA's mbarrier):
//   * full[s] lives in the first CTA (rank 0): its producer expects the bytes of BOTH CTAs' copies;
//     both producers name rank 0's barrier in their copies;
//   * empty[s] and acc_full[b] live in both CTAs: the commit that follows the MMAs arrives on both
//     (.multicast::cluster with mask 0b11); each producer / each CTA's epilogue waits on its own;
//   * acc_empty[b] lives in rank 0 and counts the epilogue warps of both CTAs (the second CTA's
//     arrive through the cluster's shared-memory window);
//   * tensor memory is allocated and freed by warp 1 of BOTH CTAs with the cta_group::2 forms, the
//     frees behind a cluster barrier.
// Waits are bounded as in the kernel above (status 121 producer, 122 / 124 MMA, 123 epilogue).
#define UP_THREADS 320
__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned mapa_u32(unsigned smem_addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar_rank0) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(dst), "l"(map), "r"(bar_rank0), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                              unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {          // arrives on `bar` of both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}

template <int EPI, int BN>
__global__ void __launch_bounds__(UP_THREADS)
gemm_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, UmmaArgs a) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_UMMA);
  constexpr int STAGE_BYTES = (UM_BM + BN / 2) * UM_BK * 2;                  // this CTA's part of a stage
  constexpr int STAGES = BN == 256 ? 6 : 8;                                  // 192 KB either way
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * STAGES + 4];           // full[], empty[], acc_full[2], acc_empty[2]
  __shared__ unsigned tmem_base_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();                                   // 0: the pair's first CTA, which issues the MMAs
  const unsigned tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const unsigned full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const unsigned accfull0 = smem_u32(&bars[2 * STAGES]), accempty0 = smem_u32(&bars[2 * STAGES + 2]);
  const unsigned full0_rank0 = mapa_u32(full0, 0), accempty0_rank0 = mapa_u32(accempty0, 0);
  const int k_blocks = (a.K + UM_BK - 1) / UM_BK;
  const int m_pairs = (a.M + 2 * UM_BM - 1) / (2 * UM_BM), n_tiles = (a.N + BN - 1) / BN, total = m_pairs * n_tiles;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accfull0 + 8 * b, 1); mbar_init(accempty0 + 8 * b, 16); }   // 8 epilogue warps of each CTA
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {                   // two accumulators of 128 x BN float32 in this CTA's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  cgx::this_cluster().sync();        // both CTAs' barriers are initialised before either names the other's
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += n_pairs) {
        const int m0 = (t % m_pairs) * 2 * UM_BM + (int)rank * UM_BM, n0 = (t / m_pairs) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(empty0 + 8 * s, (it / STAGES - 1) & 1, a.status, 121)) { ok = false; break; }
          const unsigned dst = tiles + s * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);      // the bytes of both CTAs' copies
          tma_load_2d_pair(dst, &map_a, kb * UM_BK, m0, full0_rank0 + 8 * s);
          tma_load_2d_pair(dst + UM_BM * UM_BK * 2, &map_w, kb * UM_BK, n0, full0_rank0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const unsigned idesc = umma_idesc(2 * UM_BM, BN);
      unsigned it = 0, use = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += n_pairs, ++use) {
        const unsigned acc = use & 1, d_tmem = tmem_base + acc * BN;
        if (use >= 2) {
          ok = mbar_wait(accempty0 + 8 * acc, ((use >> 1) - 1) & 1, a.status, 124);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, a.status, 122);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned sa = tiles + s * STAGE_BYTES, sb = sa + UM_BM * UM_BK * 2;
          const unsigned long long da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
          for (int k = 0; k < UM_BK / 16; ++k)
            umma_f16_pair(d_tmem, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
          umma_commit_pair(empty0 + 8 * s);             // the stage is free, in both CTAs, once these MMAs have read it
        }
        if (ok) umma_commit_pair(accfull0 + 8 * acc);   // both CTAs' epilogues
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    unsigned use = 0;
    for (int t = pair; t < total; t += n_pairs, ++use) {
      const unsigned acc = use & 1;
      const int m0 = (t % m_pairs) * 2 * UM_BM + (int)rank * UM_BM, n0 = (t / m_pairs) * BN;
      const int m = m0 + q * 32 + lane;
      constexpr int CHUNKS = BN / 2 / 32;
      constexpr int PRE = CHUNKS < 2 ? CHUNKS : 2;
      float4 res[EPI == EPI_ACC ? PRE : 1][8];
      bool res_ok[CHUNKS];
#pragma unroll
      for (int ch = 0; ch < CHUNKS; ++ch) {
        const int n = n0 + half * (BN / 2) + ch * 32;
        res_ok[ch] = EPI == EPI_ACC && ch < PRE && m < a.M && n + 32 <= a.N && (a.ldo % 4) == 0;
        if (EPI == EPI_ACC && res_ok[ch]) {
          const float4* src = (const float4*)((const float*)a.out + (size_t)m * a.ldo + n);
#pragma unroll
          for (int j = 0; j < 8; ++j) res[ch][j] = src[j];
        }
      }
      if (!mbar_wait(accfull0 + 8 * acc, (use >> 1) & 1, a.status, 123)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
      for (int ch = 0; ch < CHUNKS; ++ch) {
        const int c0 = half * (BN / 2) + ch * 32;
        float v[32];
        tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + acc * BN + (unsigned)c0, v);
        if (m < a.M && n0 + c0 < a.N) store_chunk<EPI>(a, v, m, n0 + c0, (EPI == EPI_ACC && res_ok[ch]) ? res[ch < PRE ? ch : 0] : nullptr);
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(accempty0_rank0 + 8 * acc);      // one of the sixteen arrivals that free the accumulator
    }
  }
  // common exit: every role of both CTAs comes here, also after a wait that gave up
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  cgx::this_cluster().sync();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// ---- host side: tensor maps through the driver entry point (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
// rows x K bfloat16, row stride ld elements; box = 64 k x box_rows rows, 128-byte swizzle, zeros outside
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FELLM_ERR_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {UM_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int EPI, int BN>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, const UmmaArgs& a, cudaStream_t stream) {
  size_t smem = (size_t)(BN == 256 ? 4 : UM_STAGES) * (UM_BM + BN) * UM_BK * 2 + 1024;
  auto kern = gemm_umma_kernel<EPI, BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int n_sm = fellm_sm_count();
  int total = ceil_div(a.N, BN) * ceil_div(a.M, UM_BM);
  return launch_k_class(launch_class_for_rows(a.M, 0), kern, dim3(total < n_sm ? total : n_sm, 1, 1), dim3(UM_THREADS, 1, 1), smem, stream, 1, ma, mw, a);
}

template <int EPI, int BN>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, const UmmaArgs& a, cudaStream_t stream) {
  size_t smem = (size_t)(BN == 256 ? 6 : 8) * (UM_BM + BN / 2) * UM_BK * 2 + 1024;
  auto kern = gemm_umma_pair_kernel<EPI, BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int pairs_dev = fellm_sm_count() / 2;
  const int total = ceil_div(a.N, BN) * ceil_div(a.M, 2 * UM_BM);
  const int pairs = total < pairs_dev ? total : pairs_dev;
  return launch_k_class(launch_class_for_rows(a.M, 0), kern, dim3(2 * pairs, 1, 1), dim3(UP_THREADS, 1, 1), smem, stream, 2, ma, mw, a);
}

template <int EPI>
static int launch_ksplit(const CUtensorMap& ma, const CUtensorMap& mw, const UmmaArgs& a, cudaStream_t stream) {
  const size_t smem = (size_t)UK_STAGES * (UM_BM + 128) * UM_BK * 2 + (size_t)UM_BM * UK_RECV_LD * sizeof(float) + 1024;
  auto kern = gemm_umma_ksplit_kernel<EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int total = ceil_div(a.N, 128) * ceil_div(a.M, UM_BM);
  return launch_k_class(launch_class_for_rows(a.M, 0), kern, dim3(2 * total, 1, 1), dim3(UM_THREADS, 1, 1), smem, stream, 2, ma, mw, a);
}

// status: device int32 that a role sets (101 producer, 102/104 MMA, 103 epilogue) if a wait ran out.
FELLM_API int fellm_gemm_umma(const void* A, const void* W, const float* bias, void* out, int epi, int M, int N, int K,
                              int lda, int ldw, int ldo, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!A || !W || !out || K <= 0) return FELLM_ERR_ARG;
  // TMA: 16-byte aligned bases and row strides
  if ((K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && ((N % 16) || (ldo % 8))) return FELLM_ERR_SIZE;
  // The tile: 128 x 128 or 128 x 256 by one CTA, or 256 x 256 / 256 x 128 by a CTA pair.  Chosen by an
  // estimate: waves x k-blocks x the time a CTA takes for a k-block of its tile (measured on B200 at
  // 2,048 rows: 0.37 us for 128 x 128, 0.47 us for 128 x 256, 0.44 us and 0.39 us for a pair's CTA on
  // 256 x 256 and 256 x 128) + 4.5 us of filling and draining; within 5% one CTA a tile stays.
  // FELLM_B200_UMMA_PAIR=0: never pairs; =128 / =256: always that pair tile; FELLM_B200_UMMA_WIDE=0: no 128 x 256.
  const int m_tiles = ceil_div(M, UM_BM), m_pairs = ceil_div(M, 2 * UM_BM), kb = ceil_div(K, UM_BK);
  const int n_sm = fellm_sm_count(), pairs_dev = n_sm / 2;
  static int wide_ok = -1, pair_mode = -1;
  if (wide_ok < 0) { const char* ev = getenv("FELLM_B200_UMMA_WIDE"); wide_ok = (ev && ev[0] == '0') ? 0 : 1; }
  if (pair_mode < 0) { const char* ev = getenv("FELLM_B200_UMMA_PAIR"); pair_mode = ev ? atoi(ev) : 1; }
  auto estimate = [&](int tiles, int units, float t_kb) { return 4.5f + (float)ceil_div(tiles, units) * kb * t_kb; };
  float best = estimate(ceil_div(N, 128) * m_tiles, n_sm, 0.37f);
  int choice = 0;                                           // 0: 128 x 128, 1: 128 x 256, 2: pair 256 x 256, 3: pair 256 x 128
  if (wide_ok && N >= 512) {
    const float t = estimate(ceil_div(N, 256) * m_tiles, n_sm, 0.47f);
    if (t < best) { best = t; choice = 1; }
  }
  if (pair_mode && M >= 512 && pairs_dev >= 1) {
    if (N >= 256) {
      const float t = estimate(ceil_div(N, 256) * m_pairs, pairs_dev, 0.44f);
      if (t < 0.95f * best) { best = t; choice = 2; }
    }
    const float t = estimate(ceil_div(N, 128) * m_pairs, pairs_dev, 0.39f);
    if (t < 0.95f * best) { best = t; choice = 3; }
    if (pair_mode == 256 && N >= 256) choice = 2;
    if (pair_mode == 128) choice = 3;
  }
  CUtensorMap ma, mw;
  int e = make_map(&ma, A, M, K, lda, UM_BM);
  if (e) return e;
  UmmaArgs a; a.bias = bias; a.out = out; a.status = status; a.M = M; a.N = N; a.K = K; a.ldo = ldo;
  // few tiles and a long K (a few hundred rows, a narrow N): two CTAs a 128 x 128 tile, half of K each
  static int ksplit = -1;
  if (ksplit < 0) { const char* ev = getenv("FELLM_B200_UMMA_KSPLIT"); ksplit = (ev && ev[0] == '0') ? 0 : 1; }
  if (ksplit && 2 * ceil_div(N, 128) * m_tiles <= n_sm && kb >= 8) {
    e = make_map(&mw, W, N, K, ldw, 128);
    if (e) return e;
    switch (epi) {
      case EPI_STORE: return launch_ksplit<EPI_STORE>(ma, mw, a, stream);
      case EPI_ACC: return launch_ksplit<EPI_ACC>(ma, mw, a, stream);
      case EPI_SWIGLU: return launch_ksplit<EPI_SWIGLU>(ma, mw, a, stream);
      case EPI_F32: return launch_ksplit<EPI_F32>(ma, mw, a, stream);
      default: return FELLM_ERR_ARG;
    }
  }
  if (choice >= 2) {
    const bool bn256 = choice == 2;
    e = make_map(&mw, W, N, K, ldw, bn256 ? 128 : 64);           // a CTA's half of the tile's W rows
    if (e) return e;
    switch (epi) {
      case EPI_STORE: return bn256 ? launch_pair<EPI_STORE, 256>(ma, mw, a, stream) : launch_pair<EPI_STORE, 128>(ma, mw, a, stream);
      case EPI_ACC: return bn256 ? launch_pair<EPI_ACC, 256>(ma, mw, a, stream) : launch_pair<EPI_ACC, 128>(ma, mw, a, stream);
      case EPI_SWIGLU: return bn256 ? launch_pair<EPI_SWIGLU, 256>(ma, mw, a, stream) : launch_pair<EPI_SWIGLU, 128>(ma, mw, a, stream);
      case EPI_F32: return bn256 ? launch_pair<EPI_F32, 256>(ma, mw, a, stream) : launch_pair<EPI_F32, 128>(ma, mw, a, stream);
      default: return FELLM_ERR_ARG;
    }
  }
  const bool wide = choice == 1;
  e = make_map(&mw, W, N, K, ldw, wide ? 256 : 128);
  if (e) return e;
  switch (epi) {
    case EPI_STORE: return wide ? launch<EPI_STORE, 256>(ma, mw, a, stream) : launch<EPI_STORE, 128>(ma, mw, a, stream);
    case EPI_ACC: return wide ? launch<EPI_ACC, 256>(ma, mw, a, stream) : launch<EPI_ACC, 128>(ma, mw, a, stream);
    case EPI_SWIGLU: return wide ? launch<EPI_SWIGLU, 256>(ma, mw, a, stream) : launch<EPI_SWIGLU, 128>(ma, mw, a, stream);
    case EPI_F32: return wide ? launch<EPI_F32, 256>(ma, mw, a, stream) : launch<EPI_F32, 128>(ma, mw, a, stream);
    default: return FELLM_ERR_ARG;
  }
}

// ------------------------------------------------------------------------------------------------
// Few rows (a decode step of 17..128 requests): the product is bound by reading W once, and a
// 128-row MMA fed with a few tokens would be mostly empty.  So the operands change places:
// D[n, t] = sum_k W[n, k] x[t, k], the 128 rows of the MMA are WEIGHT rows, its N the step's tokens
// (16..128 columns of tensor memory).  A CTA owns one tile of 128 weight rows and one slice of K;
// the slices of a tile are the ranks of a cluster (1, 2, 4 or 8), enough of them to spread the matrix
// over the SMs.  The TMA thread asks for the tile's weights BEFORE it waits for the kernel in
// front (they do not depend on it), for x after.  Token t of the tile belongs to rank t % S: every
// rank stores its partial sums of that token into the owner's shared memory (distributed shared
// memory stores: nobody waits for a remote load), and after ONE cluster barrier the owner adds the
// S partial rows in rank order and runs the epilogue, a warp a token, a lane four consecutive
// outputs.
//
// Roles (256 threads): warp 0 lane 0 = TMA, warp 1 = tensor memory + MMA (lane 0); once the
// products are done all eight warps read the accumulator (TMEM lane quarter = warp % 4, 16-column
// chunks by turns of warp / 4) and then share the owner's tokens.  All waits are bounded (status 111 TMA, 112 MMA,
// 113 accumulator); a role that gives up still goes through the cluster barrier.
#define SW_THREADS 256
#define SW_WARPS 8
#define SW_W_BYTES (UM_BM * UM_BK * 2)          // 16 KB: 128 weight rows x 64 k
#define SW_MAX_STAGES 12
#define SW_MAX_ROWS 128                         // tokens of a step this kernel takes

struct SwapArgs {
  const float* bias; void* out; int* status;
  int M, N, K, ldo, mt, splits, stages;         // mt: token columns of the MMA (a multiple of 16, 16..128)
  const void* next_w; long long next_bytes;     // the next product's weights, asked into L2 (or null)
  // EPI_ACC as the producer of the next RMSNorm's input (nn_x null: not asked for; N a multiple of 128): beside
  // out += ..., nn_x[t, n] = bfloat16(out[t, n] * nn_w[n]) and nn_ssq[t * (N / 128) + tile] = the sum of
  // out[t, n]^2 over the tile's 128 columns
  const float* nn_w; bf16* nn_x; float* nn_ssq; int nn_ldx;
  // ... and its consumer (rs_ssq null: none): x is such an nn_x; the finished sums of token t are multiplied by
  // 1 / sqrt(sum_p rs_ssq[t * rs_parts + p] / K + rs_eps) before the bias: RMSNorm(x) W^T with the row's
  // factor taken out of the product (crates/backend-cpu/src/kernels/norm.rs:6-39 has the norm)
  const float* rs_ssq; int rs_parts; float rs_eps;
  // EPI_CONV: the gated short convolution behind a ShortConv mixer's input product in a decode step (every token a
  // request of its own).  W's rows come in blocks of 16 B / 16 C / 16 X rows of 16 channels; a tile is two such blocks
  // (96 rows); out is y bfloat16 [M, N / 3]; the state of token t is conv_state + row_slot[t] * conv_slot_stride,
  // [taps - 1][N / 3] float32, and moves on by one token.
  const float* conv_w; const float* conv_bias; float* conv_state; const int* row_slot; long long conv_slot_stride; int conv_taps;
};
#define SW_CONV_ROWS 96
#define SW_CONV_MAX_TAPS 4

// What the next call of fellm_gemm_umma_swap is to hand on or to take over (see SwapArgs); taken and cleared
// by every call.
struct SwapHandoff { const float* nn_w; void* nn_x; float* nn_ssq; int nn_ldx; const float* rs_ssq; int rs_parts; float rs_eps; };
static SwapHandoff g_swap_handoff = {nullptr, nullptr, nullptr, 0, nullptr, 0, 0.f};
FELLM_API int fellm_gemm_umma_next_norm(const float* nn_w, void* nn_x, int nn_ldx, float* nn_ssq) {
  g_swap_handoff.nn_w = nn_w; g_swap_handoff.nn_x = nn_x; g_swap_handoff.nn_ldx = nn_ldx; g_swap_handoff.nn_ssq = nn_ssq;
  return 0;
}
FELLM_API int fellm_gemm_umma_row_scale(const float* ssq, int parts, float eps) {
  g_swap_handoff.rs_ssq = ssq; g_swap_handoff.rs_parts = parts; g_swap_handoff.rs_eps = eps;
  return 0;
}

__device__ __forceinline__ void tmem_ld16_nowait(unsigned taddr, float* v) {
  unsigned* r = reinterpret_cast<unsigned*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ unsigned mapa_rank(unsigned smem_addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(unsigned addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}

template <int EPI, int S>
__global__ void __launch_bounds__(SW_THREADS)
gemm_umma_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, SwapArgs a) {
  FELLM_TRACE_SCOPE(TRACE_GEMM_UMMA);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * SW_MAX_STAGES + 1];     // full[], empty[], accumulator done
  __shared__ unsigned tmem_base_s;
  __shared__ float rs_scale[SW_MAX_ROWS];              // the norm factors of this rank's tokens (a.rs_ssq)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int stages = a.stages, stage_bytes = SW_W_BYTES + a.mt * UM_BK * 2;
  // behind the stages: what the ranks send this CTA, [token of mine][rank][128 weight rows] float32
  float* recv = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + (size_t)stages * stage_bytes);
  const unsigned full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[SW_MAX_STAGES]), accfull = smem_u32(&bars[2 * SW_MAX_STAGES]);
  const int split = S > 1 ? (int)cgx::this_cluster().block_rank() : 0;
  // EPI_CONV: a tile is 96 weight rows (two blocks of 16 channels' B, C and X rows); the MMA still spans 128 rows,
  // the last 32 of which read whatever the stage holds there and are never looked at
  constexpr int TILE_ROWS = EPI == EPI_CONV ? SW_CONV_ROWS : UM_BM;
  const int n0 = blockIdx.y * TILE_ROWS;
  const int tx_bytes = TILE_ROWS * UM_BK * 2 + a.mt * UM_BK * 2;       // what the two copies of a stage bring
  const int kb_total = (a.K + UM_BK - 1) / UM_BK;
  const int kb0 = (int)((long long)kb_total * split / S), kb1 = (int)((long long)kb_total * (split + 1) / S);
  const int nkb = kb1 - kb0;
  const unsigned tmem_cols = a.mt <= 32 ? 32u : (a.mt <= 64 ? 64u : 128u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(accfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  pdl_launch_dependents();
  // a rank's shared memory may be written only once the rank runs: everybody says so here and
  // looks for the others' word before the first remote store (by then it has long been given)
  if (S > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");

  // the owner's part of the epilogue: warp w takes my tokens w, w + 8, ...; lane l the outputs 4l..4l+3
  const int my_tokens = split < a.M ? (a.M - split + S - 1) / S : 0;
  float4 res[2];                                    // += residual: fetched while the products run (up to 16 tokens a rank)
  bool res_ok[2] = {false, false};
  float4 nn_g = make_float4(0.f, 0.f, 0.f, 0.f);    // the next norm's weights of this lane's four columns
  if (EPI == EPI_ACC && a.nn_x) nn_g = *(const float4*)(a.nn_w + n0 + 4 * lane);
  // EPI_CONV: lanes 0..3 and 12..15 hold the B rows of four channels each (C: four lanes on, X: eight lanes on); they
  // run the convolution of those channels and ask for the taps now
  const bool conv_lane = EPI == EPI_CONV && lane < 24 && (lane % 12) < 4;
  const int conv_ch = n0 / 3 + 16 * (lane / 12) + 4 * (lane % 12);         // first of the lane's four channels
  float cw[EPI == EPI_CONV ? 4 : 1][SW_CONV_MAX_TAPS], cb[4] = {0.f, 0.f, 0.f, 0.f};
  if (EPI == EPI_CONV && conv_lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int tt = 0; tt < SW_CONV_MAX_TAPS; ++tt) cw[c][tt] = tt < a.conv_taps ? a.conv_w[(size_t)(conv_ch + c) * a.conv_taps + tt] : 0.f;
      if (a.conv_bias) cb[c] = a.conv_bias[conv_ch + c];
    }
  }

  if (warp == 0 && lane == 0) {
    // weights first: they do not depend on the kernel in front
    const int first = nkb < stages ? nkb : stages;
    for (int i = 0; i < first; ++i) {
      mbar_expect_tx(full0 + 8 * i, tx_bytes);
      tma_load_2d(tiles + i * stage_bytes, &map_w, (kb0 + i) * UM_BK, n0, full0 + 8 * i);
    }
    l2_prefetch_share(a.next_w, a.next_bytes, blockIdx.y * S + blockIdx.x, gridDim.y * S);
    pdl_wait(); FELLM_TRACE_WAITED();
    for (int i = 0; i < first; ++i)
      tma_load_2d(tiles + i * stage_bytes + SW_W_BYTES, &map_x, (kb0 + i) * UM_BK, 0, full0 + 8 * i);
    for (int it = first; it < nkb; ++it) {
      const int s = it % stages;
      if (!mbar_wait(empty0 + 8 * s, (it / stages - 1) & 1, a.status, 111)) break;
      mbar_expect_tx(full0 + 8 * s, tx_bytes);
      tma_load_2d(tiles + s * stage_bytes, &map_w, (kb0 + it) * UM_BK, n0, full0 + 8 * s);
      tma_load_2d(tiles + s * stage_bytes + SW_W_BYTES, &map_x, (kb0 + it) * UM_BK, 0, full0 + 8 * s);
    }
#ifdef FELLM_TRACE
    FELLM_TRACE_MARK(0);                                     // every load asked for
    mbar_wait(accfull, 0, nullptr, 0);
    FELLM_TRACE_MARK(1);                                     // the tile's products done
#endif
  } else {
    pdl_wait();                      // what the other threads read of global memory (out, for +=) the kernel in front wrote
    if (warp == 1 && lane == 0) {
      const unsigned idesc = umma_idesc(UM_BM, a.mt);
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        const int s = it % stages;
        ok = mbar_wait(full0 + 8 * s, (it / stages) & 1, a.status, 112);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned sw = tiles + s * stage_bytes, sx = sw + SW_W_BYTES;
        const unsigned long long dw = umma_desc(sw), dx = umma_desc(sx);
#pragma unroll
        for (int k = 0; k < UM_BK / 16; ++k)
          umma_f16(tmem_base, dw + (unsigned long long)(k * 2), dx + (unsigned long long)(k * 2), idesc, (it | k) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);
      }
      if (ok) umma_commit(accfull);
    } else if (warp >= 2 && a.rs_ssq) {
      // the other warps have nothing to do until the products are done: the norm factors of this rank's
      // tokens, the parts of a row always added in the same order
      for (int tl = warp - 2; tl < my_tokens; tl += SW_WARPS - 2) {
        const float* parts = a.rs_ssq + (size_t)(split + tl * S) * a.rs_parts;
        float ss = 0.f;
        for (int p = lane; p < a.rs_parts; p += 32) ss += parts[p];
        ss = warp_sum(ss);
        if (lane == 0) rs_scale[tl] = 1.0f / sqrtf(ss / (float)a.K + a.rs_eps);
      }
    }
  }
  __syncwarp();
  if (S > 1) asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
  if (EPI == EPI_ACC && (a.ldo % 4) == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int tl = warp + SW_WARPS * i, n = n0 + 4 * lane;
      if (tl < my_tokens && n + 4 <= a.N) {
        res[i] = *(const float4*)((const float*)a.out + (size_t)(split + tl * S) * a.ldo + n);
        res_ok[i] = true;
      }
    }
  }
  {
    const int q = warp & 3, row = q * 32 + lane;
    const bool done = mbar_wait(accfull, 0, a.status, 113);
    __syncwarp();
    if (done && (EPI != EPI_CONV || q < 3)) {                  // (EPI_CONV: rows 96..127 are nobody's)
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      // token t goes to rank t % S, slot [t / S][my rank][row] there
      const unsigned recv0 = smem_u32(recv);
      unsigned dst_rank[S];
#pragma unroll
      for (int j = 0; j < S; ++j) dst_rank[j] = S > 1 ? mapa_rank(recv0, (unsigned)j) : recv0;
      for (int c0 = 16 * (warp >> 2); c0 < a.mt; c0 += 32) {
        float v[16];
        tmem_ld16_nowait(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = c0 + j;                    // c0 is a multiple of 16, S divides 16: the owner is j % S
          if (t < a.M) st_cluster_f32(dst_rank[j % S] + (unsigned)((((t / S) * S + split) * UM_BM + row) * 4), v[j]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  if (S > 1) cgx::this_cluster().sync(); else __syncthreads();      // the remote stores are visible behind it
  FELLM_TRACE_MARK(2);

  auto finish = [&](int tl, float4 v, bool have_res, const float4& res_i) {
    const int t = split + tl * S, n = n0 + 4 * lane;
    if (a.rs_ssq) { const float sc = rs_scale[tl]; v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc; }
    if (a.bias) {
      if (n < a.N) v.x += a.bias[n];
      if (n + 1 < a.N) v.y += a.bias[n + 1];
      if (n + 2 < a.N) v.z += a.bias[n + 2];
      if (n + 3 < a.N) v.w += a.bias[n + 3];
    }
    if (EPI == EPI_CONV) {
      // B, C and X as the stored product would round them; bx = B*X; conv = bx*w[Lc-1] + sum_t state[t]*w[t]
      // (oldest first); y = C*(conv + bias); the state moves on by one (crates/backend-cpu/src/kernels/shortconv.rs:61-106)
      v.x = __bfloat162float(__float2bfloat16_rn(v.x)); v.y = __bfloat162float(__float2bfloat16_rn(v.y));
      v.z = __bfloat162float(__float2bfloat16_rn(v.z)); v.w = __bfloat162float(__float2bfloat16_rn(v.w));
      float cv[4], xv[4];
      cv[0] = __shfl_down_sync(0xffffffffu, v.x, 4); cv[1] = __shfl_down_sync(0xffffffffu, v.y, 4);
      cv[2] = __shfl_down_sync(0xffffffffu, v.z, 4); cv[3] = __shfl_down_sync(0xffffffffu, v.w, 4);
      xv[0] = __shfl_down_sync(0xffffffffu, v.x, 8); xv[1] = __shfl_down_sync(0xffffffffu, v.y, 8);
      xv[2] = __shfl_down_sync(0xffffffffu, v.z, 8); xv[3] = __shfl_down_sync(0xffffffffu, v.w, 8);
      if (conv_lane) {
        const int H = a.conv_taps - 1, d = a.N / 3;
        float* st = a.conv_state + (size_t)a.row_slot[t] * a.conv_slot_stride + conv_ch;
        float4 hist[SW_CONV_MAX_TAPS - 1];
#pragma unroll
        for (int tt = 0; tt < SW_CONV_MAX_TAPS - 1; ++tt) hist[tt] = tt < H ? *(const float4*)(st + (size_t)tt * d) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float bv[4] = {v.x, v.y, v.z, v.w};
        float bx[4], y[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          bx[c] = bv[c] * xv[c];
          float wlast = 0.f;
#pragma unroll
          for (int tt = 0; tt < SW_CONV_MAX_TAPS; ++tt) if (tt == H) wlast = cw[c][tt];
          float conv = bx[c] * wlast;
#pragma unroll
          for (int tt = 0; tt < SW_CONV_MAX_TAPS - 1; ++tt) {
            const float hc = c == 0 ? hist[tt].x : (c == 1 ? hist[tt].y : (c == 2 ? hist[tt].z : hist[tt].w));
            if (tt < H) conv = fmaf(hc, cw[c][tt], conv);
          }
          y[c] = cv[c] * (conv + cb[c]);
        }
        const __nv_bfloat162 y0 = __floats2bfloat162_rn(y[0], y[1]), y1 = __floats2bfloat162_rn(y[2], y[3]);
        *(uint2*)((bf16*)a.out + (size_t)t * a.ldo + conv_ch) = make_uint2(*(const unsigned*)&y0, *(const unsigned*)&y1);
#pragma unroll
        for (int tt = 0; tt < SW_CONV_MAX_TAPS - 1; ++tt) {
          if (tt < H) *(float4*)(st + (size_t)tt * d) = (tt + 1 < H) ? hist[tt + 1 < SW_CONV_MAX_TAPS - 1 ? tt + 1 : tt] : make_float4(bx[0], bx[1], bx[2], bx[3]);
        }
      }
    } else if (EPI == EPI_SWIGLU) {
      // rows in blocks of 16: 8 gate, then the 8 up rows of the same features: lanes 4b+2, 4b+3 hold the up values of lanes 4b, 4b+1
      float4 up;
      up.x = __shfl_down_sync(0xffffffffu, v.x, 2); up.y = __shfl_down_sync(0xffffffffu, v.y, 2);
      up.z = __shfl_down_sync(0xffffffffu, v.z, 2); up.w = __shfl_down_sync(0xffffffffu, v.w, 2);
      if ((lane & 3) < 2 && n < a.N) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn((v.x / (1.0f + expf(-v.x))) * up.x, (v.y / (1.0f + expf(-v.y))) * up.y);
        __nv_bfloat162 p1 = __floats2bfloat162_rn((v.z / (1.0f + expf(-v.z))) * up.z, (v.w / (1.0f + expf(-v.w))) * up.w);
        bf16* dst = (bf16*)a.out + (size_t)t * a.ldo + ((n0 + 16 * (lane >> 2)) >> 1) + 4 * (lane & 1);
        if ((a.ldo % 4) == 0) *(uint2*)dst = make_uint2(*(unsigned*)&p0, *(unsigned*)&p1);
        else { dst[0] = p0.x; dst[1] = p0.y; dst[2] = p1.x; dst[3] = p1.y; }
      }
    } else if (n + 4 <= a.N && (a.ldo % 4) == 0) {
      const size_t o = (size_t)t * a.ldo + n;
      if (EPI == EPI_STORE) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v.x, v.y), p1 = __floats2bfloat162_rn(v.z, v.w);
        *(uint2*)((bf16*)a.out + o) = make_uint2(*(unsigned*)&p0, *(unsigned*)&p1);
      } else {
        if (EPI == EPI_ACC) {
          const float4 r = have_res ? res_i : *(const float4*)((const float*)a.out + o);
          v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
          if (a.nn_x) {
            // (N is a multiple of 128 here: the whole warp is in this branch)
            const float sq = warp_sum(fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))));
            const __nv_bfloat162 g0 = __floats2bfloat162_rn(v.x * nn_g.x, v.y * nn_g.y), g1 = __floats2bfloat162_rn(v.z * nn_g.z, v.w * nn_g.w);
            *(uint2*)(a.nn_x + (size_t)t * a.nn_ldx + n) = make_uint2(*(const unsigned*)&g0, *(const unsigned*)&g1);
            if (lane == 0) a.nn_ssq[(size_t)t * gridDim.y + blockIdx.y] = sq;
          }
        }
        *(float4*)((float*)a.out + o) = v;
      }
    } else {
      const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (n + c >= a.N) break;
        const size_t o = (size_t)t * a.ldo + n + c;
        if (EPI == EPI_STORE) ((bf16*)a.out)[o] = __float2bfloat16_rn(e[c]);
        else if (EPI == EPI_ACC) ((float*)a.out)[o] += e[c];
        else ((float*)a.out)[o] = e[c];
      }
    }
  };
  // two tokens a turn: their 2 S partial rows are asked for together, summed in rank order
#pragma unroll 1
  for (int tl0 = warp; tl0 < my_tokens; tl0 += 2 * SW_WARPS) {
    float4 p[2][S];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int tl = tl0 + SW_WARPS * u;
      if (tl < my_tokens) {
        const float4* rows = reinterpret_cast<const float4*>(recv + (size_t)tl * S * UM_BM) + lane;
#pragma unroll
        for (int j = 0; j < S; ++j) p[u][j] = rows[j * (UM_BM / 4)];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int tl = tl0 + SW_WARPS * u;
      if (tl < my_tokens) {
        float4 v = p[u][0];
#pragma unroll
        for (int j = 1; j < S; ++j) { v.x += p[u][j].x; v.y += p[u][j].y; v.z += p[u][j].z; v.w += p[u][j].w; }
        finish(tl, v, tl0 == warp && res_ok[u], res[u]);
      }
    }
  }
  FELLM_TRACE_MARK(3);
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

struct SwapPlan { int mt, splits, stages; size_t smem; };
static int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return (e && e[0]) ? atoi(e) : dflt;
}
template <int EPI, int S>
static int launch_swap_s(const CUtensorMap& mw, const CUtensorMap& mx, const SwapArgs& a, size_t smem, int n_tiles, cudaStream_t stream) {
  auto kern = gemm_umma_swap_kernel<EPI, S>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return launch_k_class(1, kern, dim3(S, n_tiles, 1), dim3(SW_THREADS, 1, 1), smem, stream, S, mw, mx, a);
}
template <int EPI>
static int launch_swap(const CUtensorMap& mw, const CUtensorMap& mx, const SwapArgs& a, size_t smem, int n_tiles, cudaStream_t stream) {
  switch (a.splits) {
    case 1: return launch_swap_s<EPI, 1>(mw, mx, a, smem, n_tiles, stream);
    case 2: return launch_swap_s<EPI, 2>(mw, mx, a, smem, n_tiles, stream);
    case 4: return launch_swap_s<EPI, 4>(mw, mx, a, smem, n_tiles, stream);
    case 8: return launch_swap_s<EPI, 8>(mw, mx, a, smem, n_tiles, stream);
    default: return FELLM_ERR_SIZE;
  }
}

// Clusters of S CTAs with `smem` bytes each that the device holds at once (a cluster's CTAs sit in one GPC,
// so this is less than SMs / S where a CTA fills an SM).  The += kernel stands for all epilogues (the same
// resources).  Asked once per (device, S, KB of shared memory).
template <int S>
static int swap_max_clusters(size_t smem) {
  static int cache[8][256];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 8) dev = 0;
  const int kb = (int)(smem / 1024) < 255 ? (int)(smem / 1024) : 255;
  if (!cache[dev][kb]) {
    auto kern = gemm_umma_swap_kernel<EPI_ACC, S>;
    int n = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(S, 4096, 1); cfg.blockDim = dim3(SW_THREADS, 1, 1); cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = S; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr; cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
    }
    cache[dev][kb] = n > 0 ? n : fellm_sm_count() / S / 2;      // no answer (no device here): a careful guess
    if (cache[dev][kb] < 1) cache[dev][kb] = 1;
  }
  return cache[dev][kb];
}

// One CTA to an SM with most of its shared memory as weight stages (measured on B200, a decode step of
// 64 rows at width 1024: 0.93 ms with 128..200 KB a CTA against 1.02 ms with two CTAs of 100 KB to an SM);
// as many K slices (8, 4, 2, 1: the ranks of a cluster) as keep the tile's clusters in ONE wave: with
// clusters of 8 CTAs that fill their SMs a B200 holds fewer than 148 / 8 of them, and a second wave
// doubled the time of the [2048, 2048] product at 64 rows.
static void plan_swap_s(int M, int N, int K, int splits, SwapPlan* p) {
  static int budget_kb = 0;
  if (!budget_kb) budget_kb = env_int("FELLM_B200_SWAP_SMEM_KB", 160);
  const int kb_total = ceil_div(K, UM_BK);
  p->mt = ceil_div(M, 16) * 16;
  p->splits = splits;
  const int stage_bytes = SW_W_BYTES + p->mt * UM_BK * 2;
  const size_t recv = (size_t)ceil_div(p->mt, splits) * splits * UM_BM * sizeof(float);
  int stages = ceil_div(kb_total, splits);
  const int budget = p->mt > 64 ? 220 : budget_kb;            // (more than 64 tokens: their partial rows alone take up to 64 KB)
  int fit = (int)(((size_t)budget * 1024 - 1024 - recv) / stage_bytes);
  if (fit < 2) fit = 2;
  if (stages > fit) stages = fit;
  if (stages > SW_MAX_STAGES) stages = SW_MAX_STAGES;
  p->stages = stages;
  p->smem = (size_t)stages * stage_bytes + recv + 1024;
}
static bool plan_swap(int M, int N, int K, SwapPlan* p, int tile_rows = UM_BM) {
  if (M < 1 || M > SW_MAX_ROWS || K % 8) return false;
  static int max_splits = 0;
  if (!max_splits) max_splits = env_int("FELLM_B200_SWAP_SPLITS", 8);
  const int n_sm = fellm_sm_count();
  const int n_tiles = ceil_div(N, tile_rows), kb_total = ceil_div(K, UM_BK);
  for (int splits = 8; splits > 1; splits /= 2) {
    if (splits > max_splits || splits > kb_total || n_tiles * splits > n_sm) continue;
    plan_swap_s(M, N, K, splits, p);
    const int room = splits == 8 ? swap_max_clusters<8>(p->smem) : (splits == 4 ? swap_max_clusters<4>(p->smem) : swap_max_clusters<2>(p->smem));
    if (room >= n_tiles) return true;
  }
  plan_swap_s(M, N, K, 1, p);
  return true;
}

// Whether fellm_gemm_umma_swap takes the product (1) or not (0).
FELLM_API int fellm_gemm_umma_swap_takes(int M, int N, int K) {
  SwapPlan p;
  return (M >= 1 && M <= SW_MAX_ROWS && N >= 1 && K >= 8 && plan_swap(M, N, K, &p)) ? 1 : 0;
}

// out[M, N] = x[M, K] W[N, K]^T for M <= 128 rows with the operands' places changed (see above).
// Same epilogues and status word as fellm_gemm_umma (111..113 for this kernel's roles).
FELLM_API int fellm_gemm_umma_swap(const void* x, const void* W, const float* bias, void* out, int epi, int M, int N, int K,
                                   int lda, int ldw, int ldo, int* status, cudaStream_t stream) {
  const SwapHandoff h = g_swap_handoff;                  // taken and cleared whatever this call returns
  g_swap_handoff = SwapHandoff{nullptr, nullptr, nullptr, 0, nullptr, 0, 0.f};
  const NextWeights nw = take_next_weights();
  if (M <= 0 || N <= 0) return 0;
  if (!x || !W || !out || K <= 0) return FELLM_ERR_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return FELLM_ERR_SIZE;
  if (epi == EPI_SWIGLU && (N % 16)) return FELLM_ERR_SIZE;
  SwapPlan p;
  if (!plan_swap(M, N, K, &p)) return FELLM_ERR_SIZE;
  if (h.nn_x && (epi != EPI_ACC || !h.nn_w || !h.nn_ssq || (N % UM_BM) || (ldo % 4) || (h.nn_ldx % 4) || h.nn_ldx < N ||
                 ((uintptr_t)h.nn_x & 7) || ((uintptr_t)h.nn_w & 15))) return FELLM_ERR_ARG;
  if (h.rs_ssq && h.rs_parts < 1) return FELLM_ERR_ARG;
  CUtensorMap mw, mx;
  int e = make_map(&mw, W, N, K, ldw, UM_BM);
  if (e) return e;
  e = make_map(&mx, x, M, K, lda, p.mt);
  if (e) return e;
  SwapArgs a = {};
  a.bias = bias; a.out = out; a.status = status; a.M = M; a.N = N; a.K = K; a.ldo = ldo;
  a.mt = p.mt; a.splits = p.splits; a.stages = p.stages;
  a.next_w = nw.ptr; a.next_bytes = nw.bytes;
  a.nn_w = h.nn_w; a.nn_x = (bf16*)h.nn_x; a.nn_ssq = h.nn_ssq; a.nn_ldx = h.nn_ldx;
  a.rs_ssq = h.rs_ssq; a.rs_parts = h.rs_parts; a.rs_eps = h.rs_eps;
  const int n_tiles = ceil_div(N, UM_BM);
  switch (epi) {
    case EPI_STORE: return launch_swap<EPI_STORE>(mw, mx, a, p.smem, n_tiles, stream);
    case EPI_ACC: return launch_swap<EPI_ACC>(mw, mx, a, p.smem, n_tiles, stream);
    case EPI_SWIGLU: return launch_swap<EPI_SWIGLU>(mw, mx, a, p.smem, n_tiles, stream);
    case EPI_F32: return launch_swap<EPI_F32>(mw, mx, a, p.smem, n_tiles, stream);
    default: return FELLM_ERR_ARG;
  }
}

// A decode step's ShortConv input product and gated convolution in one launch, for 17..128 tokens (every token a
// request of its own; fellm_gemm_skinny_conv is the same for up to 16): W [3d, K] with its rows in blocks of 16 B /
// 16 C / 16 X rows of 16 channels, d a multiple of 32, 2..4 taps; y bfloat16 [M, d]; state float32, slot_stride floats
// between slots, row_slot[t] the slot of token t.  x may be the weighted rows of a handed-on norm
// (fellm_gemm_umma_row_scale before the call).  FELLM_ERR_SIZE for what it does not take (fellm_gemm_umma_swap_conv_takes).
static bool swap_conv_ok(int M, int N, int K, int taps) {
  return M >= 1 && M <= SW_MAX_ROWS && N > 0 && N % SW_CONV_ROWS == 0 && K >= 8 && K % 8 == 0 && taps >= 2 && taps <= SW_CONV_MAX_TAPS;
}
FELLM_API int fellm_gemm_umma_swap_conv_takes(int M, int N, int K, int taps) {
  SwapPlan p;
  return (swap_conv_ok(M, N, K, taps) && plan_swap(M, N, K, &p, SW_CONV_ROWS)) ? 1 : 0;
}
FELLM_API int fellm_gemm_umma_swap_conv(const void* x, const void* W, const float* bias, const float* conv_w, const float* conv_bias,
                                        float* state, long long slot_stride, const int* row_slot, int taps, void* y,
                                        int M, int N, int K, int lda, int ldw, int ldy, int* status, cudaStream_t stream) {
  const SwapHandoff h = g_swap_handoff;                  // taken and cleared whatever this call returns
  g_swap_handoff = SwapHandoff{nullptr, nullptr, nullptr, 0, nullptr, 0, 0.f};
  const NextWeights nw = take_next_weights();
  if (M <= 0 || N <= 0) return 0;
  if (!x || !W || !y || !conv_w || !state || !row_slot || K <= 0) return FELLM_ERR_ARG;
  if (!swap_conv_ok(M, N, K, taps) || (lda % 8) || (ldw % 8) || (ldy % 4) || (slot_stride % 4) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15) ||
      ((uintptr_t)state & 15) || ((uintptr_t)y & 7)) return FELLM_ERR_SIZE;
  if (h.nn_x) return FELLM_ERR_ARG;
  if (h.rs_ssq && h.rs_parts < 1) return FELLM_ERR_ARG;
  SwapPlan p;
  if (!plan_swap(M, N, K, &p, SW_CONV_ROWS)) return FELLM_ERR_SIZE;
  CUtensorMap mw, mx;
  int e = make_map(&mw, W, N, K, ldw, SW_CONV_ROWS);
  if (e) return e;
  e = make_map(&mx, x, M, K, lda, p.mt);
  if (e) return e;
  SwapArgs a = {};
  a.bias = bias; a.out = y; a.status = status; a.M = M; a.N = N; a.K = K; a.ldo = ldy;
  a.mt = p.mt; a.splits = p.splits; a.stages = p.stages;
  a.next_w = nw.ptr; a.next_bytes = nw.bytes;
  a.rs_ssq = h.rs_ssq; a.rs_parts = h.rs_parts; a.rs_eps = h.rs_eps;
  a.conv_w = conv_w; a.conv_bias = conv_bias; a.conv_state = state; a.row_slot = row_slot; a.conv_slot_stride = slot_stride;
  a.conv_taps = taps;
  return launch_swap<EPI_CONV>(mw, mx, a, p.smem, N / SW_CONV_ROWS, stream);
}

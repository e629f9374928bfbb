// Shared device helpers for the fellm_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FELLM_API extern "C" __attribute__((visibility("default")))

// Launchers return 0 on success, a positive cudaError_t, or one of these negative codes.
#define FELLM_ERR_SIZE (-1)      // a size the kernel does not take
#define FELLM_ERR_ARG (-2)       // a null or inconsistent argument

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- programmatic dependent launch: a kernel launched with launch_k() may start while its
// predecessor in the stream is still running.  What does not depend on the predecessor (weight
// prefetch, index set-up) goes before pdl_wait(); everything that reads or writes data another
// kernel of the step touches goes after it.  pdl_wait() returns once the predecessor has completed
// and its writes are visible; it is a no-op for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- kernel timeline (built only with -DFELLM_TRACE=1): thread 0 of every CTA records the global
// timer at the kernel's entry, after pdl_wait() and at its exit into a buffer that
// fellm_set_trace() names; without the define the macros are empty.
enum TraceKernel { TRACE_EMBED_ROWS = 1, TRACE_RMSNORM, TRACE_RMSNORM_VEC, TRACE_SILU_MUL, TRACE_GEMM_SIMT, TRACE_GEMM_TILED,
                   TRACE_GEMM_UMMA, TRACE_SHORTCONV, TRACE_QK_ROPE_WRITE, TRACE_QK_ROPE_WRITE_VEC, TRACE_ATTENTION_SIMT,
                   TRACE_ATTENTION_PREFILL, TRACE_ATTENTION_DECODE, TRACE_SAMPLE, TRACE_COUNT_TOKENS, TRACE_ARGMAX_PARTIAL,
                   TRACE_ARGMAX_FINAL, TRACE_GEMM_SKINNY = 32 /* + 32 * epilogue */ };
#ifdef FELLM_TRACE
static __device__ unsigned long long* g_trace_buf;      // [capacity][8]: tag, entry, after wait, exit, 4 marks
static __device__ unsigned* g_trace_count;
static __device__ unsigned g_trace_capacity;
extern "C" __attribute__((visibility("default"))) int fellm_set_trace(void* buf, void* count, unsigned capacity) {
  cudaError_t e = cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof(buf));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_count, &count, sizeof(count));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_capacity, &capacity, sizeof(capacity));
  return (int)e;
}
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
struct TraceScope {
  unsigned long long* rec;
  __device__ __forceinline__ TraceScope(int id) : rec(nullptr) {
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0 && g_trace_buf) {
      unsigned i = atomicAdd(g_trace_count, 1u);
      if (i < g_trace_capacity) {
        rec = g_trace_buf + 8 * (size_t)i;
        unsigned long long blocks = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
        rec[0] = (unsigned long long)id | (blocks << 16);
        rec[2] = 0; rec[4] = 0; rec[5] = 0; rec[6] = 0; rec[7] = 0;
        rec[1] = trace_now();
      }
    }
  }
  __device__ __forceinline__ void waited() { if (rec) rec[2] = trace_now(); }
  __device__ __forceinline__ void mark(int k) { if (rec) rec[4 + k] = trace_now(); }
  __device__ __forceinline__ ~TraceScope() { if (rec) rec[3] = trace_now(); }
};
#define FELLM_TRACE_SCOPE(id) TraceScope fellm_trace_scope(id)
#define FELLM_TRACE_WAITED() fellm_trace_scope.waited()
#define FELLM_TRACE_MARK(k) fellm_trace_scope.mark(k)
#else
#define FELLM_TRACE_SCOPE(id) do { } while (0)
#define FELLM_TRACE_WAITED() do { } while (0)
#define FELLM_TRACE_MARK(k) do { } while (0)
#endif

#include <cstdlib>
static inline bool pdl_enabled(int launch_class) {
  static int on = -1;
  // FELLM_B200_PDL: 0 = never; 2 (the default) = only launches of class 1, the weight-streaming
  // products, which request their weights before they wait for the kernel before them; 3 = also
  // class 2 (short element-wise kernels); 1 = every launch.  Measured on B200, one decode step of
  // 88 dependent launches replayed from a CUDA graph (batch 8, 16 layers of width 1024): 465 us
  // with 0, 404 us with 2, 429 us with 3, 421 us with 1: kernels with nothing to do before their
  // wait only take SM room from the kernel they wait for.
  if (on < 0) { const char* e = getenv("FELLM_B200_PDL"); on = (e && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 2; }
  return on == 1 || (on == 2 && launch_class == 1) || (on == 3 && (launch_class == 1 || launch_class == 2));
}

// Launches `kernel` with an optional cluster along x and, with FELLM_B200_PDL=1, as a
// programmatic dependent of the kernel before it.  Returns a cudaError_t as int.
template <typename... KArgs, typename... Args>
static int launch_k_class(int launch_class, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled(launch_class)) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr; cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
template <typename... KArgs, typename... Args>
static int launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                    int cluster_x, Args... args) {
  return launch_k_class(0, kernel, grid, block, smem, stream, cluster_x, args...);
}

// A step of many rows (portions of prompts) is a chain of kernels of tens of microseconds each: every
// one of them is launched as a programmatic dependent (class 1), so that a launch's gap (~2 us) and
// the kernel's set-up hide under the kernel in front (measured on B200, a prompt of 2,048 tokens
// through 16 layers of width 1024: 2.13 -> 2.05 ms).  Few rows (decode steps): the class the caller names.
#define FELLM_MANY_ROWS 128
static inline int launch_class_for_rows(long long rows, int few_rows_class) {
  return rows >= FELLM_MANY_ROWS ? 1 : few_rows_class;
}

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return (int)e;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// SMs of the current device (asked once per device; the planners size grids and waves by it).
static inline int fellm_sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;   // B200
    cached[dev] = n;
  }
  return cached[dev];
}


// ---- the next product's weights into L2.  A decode step is a chain of short dependent products, each bound
// by the latency of its own first bytes; which matrix the product AFTER this one reads is known on the
// host, so a launch can be told (fellm_next_weights, consumed by the module's next launch) and its CTAs
// then ask the L2 for that matrix, a share each, before they wait for the kernel in front: the DRAM
// stream no longer stops between kernels, and the next product finds its weights a cache hit away.
#ifdef FELLM_WEIGHT_PREFETCH
struct NextWeights { const void* ptr; long long bytes; };
static NextWeights g_next_weights = {nullptr, 0};
FELLM_API int fellm_next_weights(const void* ptr, long long bytes) {
  g_next_weights.ptr = (ptr && bytes >= 16 && !((uintptr_t)ptr & 15)) ? ptr : nullptr;
  g_next_weights.bytes = g_next_weights.ptr ? bytes : 0;
  return 0;
}
static inline NextWeights take_next_weights() {
  NextWeights n = g_next_weights;
  g_next_weights.ptr = nullptr; g_next_weights.bytes = 0;
  return n;
}
// CTA `cta` of `n_ctas` asks for the pieces cta, cta + n_ctas, ... of 16 KB; `lane` of `lanes` of its threads take
// them in turns (one thread: lane 0 of 1).
__device__ __forceinline__ void l2_prefetch_share(const void* ptr, long long bytes, int cta, int n_ctas, int lane = 0, int lanes = 1) {
  if (!ptr) return;
  const long long piece = 16384, n = (bytes + piece - 1) / piece;
  for (long long i = cta + (long long)lane * n_ctas; i < n; i += (long long)lanes * n_ctas) {
    const long long off = i * piece;
    const unsigned size = (unsigned)((bytes - off < piece ? bytes - off : piece) & ~15ll);
    if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"((const char*)ptr + off), "r"(size) : "memory");
  }
}
#endif

// The no-allocation variant of split-KV decode attention: same kernel as attention_mma.cu, scratch
// and counters in file-scope device arrays.  See attention_decode_static.h for the contract.
#include "attention_decode_static.h"

#include <cstdio>
#include <mutex>

#include "attention_mma.cu"

static __device__ __align__(256) float g_static_scratch[FELLM_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_counters[FELLM_STATIC_COUNTERS];

// In host code the two names above are host-side stand-ins, not device addresses: the addresses a
// kernel may use come from cudaGetSymbolAddress, once per device.
#define FELLM_STATIC_MAX_DEVICES 64
static float* s_scratch_ptr[FELLM_STATIC_MAX_DEVICES];
static int* s_counter_ptr[FELLM_STATIC_MAX_DEVICES];
static bool s_ready[FELLM_STATIC_MAX_DEVICES];
static std::mutex s_mutex;

static int say(char* err, int err_len, int code, const char* fmt, long long a = 0, long long b = 0) {
  if (err && err_len > 0) snprintf(err, (size_t)err_len, fmt, a, b);
  return code;
}

FELLM_API int fellm_attn_decode_static(const void* q, const void* pool, const int* block_table, int max_pages,
                                       const int* positions, const int* row_slot, void* out, int T, int H, int G,
                                       int hd, int page_tokens, int layer, int layers_in_group, float scale,
                                       int window, int split_len, int max_splits, cudaStream_t stream, char* err,
                                       int err_len) {
  if (err && err_len > 0) err[0] = 0;
  if (T <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, q, pool, block_table, max_pages, positions, row_slot, out, T, H, G, hd, page_tokens, layer,
                    layers_in_group, scale, window);
  if (e == FELLM_ERR_SIZE)
    return say(err, err_len, e, "this library is built for head size %lld and whole groups of heads; got head size %lld", HD, hd);
  if (e) return say(err, err_len, e, "a null pointer among the arguments");
  if (split_len < 1 || max_splits < 1) return say(err, err_len, FELLM_ERR_ARG, "split_len and max_splits must be at least 1");
  long long need_f = (long long)T * H * max_splits * (HD + 2), need_c = (long long)T * G;
  if (need_f > FELLM_STATIC_SCRATCH_FLOATS)
    return say(err, err_len, FELLM_STATIC_TOO_LARGE,
               "the launch needs %lld scratch floats (rows*heads*max_splits*(head_dim+2)); the built-in array holds %lld",
               need_f, (long long)FELLM_STATIC_SCRATCH_FLOATS);
  if (need_c > FELLM_STATIC_COUNTERS)
    return say(err, err_len, FELLM_STATIC_TOO_LARGE,
               "the launch needs %lld counters (rows*kv_heads); the built-in array holds %lld", need_c,
               (long long)FELLM_STATIC_COUNTERS);

  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return say(err, err_len, (int)ce, "cudaGetDevice failed (%lld)", (long long)ce);
  if (dev < 0 || dev >= FELLM_STATIC_MAX_DEVICES) return say(err, err_len, FELLM_ERR_ARG, "device ordinal %lld is out of range", dev);
  size_t ring = (size_t)DC_WARPS * DC_STAGES * 2 * DC_TK * ROWB, mrg = (size_t)DC_WARPS * 16 * (HD + 2) * sizeof(float);
  size_t smem = ring > mrg ? ring : mrg;
  {
    std::lock_guard<std::mutex> lock(s_mutex);
    if (!s_ready[dev]) {                     // first call on this device, which is the current one
      ce = cudaGetSymbolAddress((void**)&s_scratch_ptr[dev], g_static_scratch);
      if (ce != cudaSuccess) return say(err, err_len, (int)ce, "cudaGetSymbolAddress(scratch) failed (%lld)", (long long)ce);
      ce = cudaGetSymbolAddress((void**)&s_counter_ptr[dev], g_static_counters);
      if (ce != cudaSuccess) return say(err, err_len, (int)ce, "cudaGetSymbolAddress(counters) failed (%lld)", (long long)ce);
      if (smem > 32 * 1024) {        // static shared memory counts against the 48 KB default too
        ce = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return say(err, err_len, (int)ce, "cudaFuncSetAttribute failed (%lld)", (long long)ce);
      }
      s_ready[dev] = true;
    }
  }
  a.scratch = s_scratch_ptr[dev];
  a.counters = s_counter_ptr[dev];
  a.split_len = split_len;
  a.max_splits = max_splits;
  // the counters this launch uses start at zero, whatever an earlier call left
  ce = cudaMemsetAsync(a.counters, 0, (size_t)need_c * sizeof(int), stream);
  if (ce != cudaSuccess) return say(err, err_len, (int)ce, "cudaMemsetAsync failed (%lld)", (long long)ce);
  int rc = launch_k(attention_decode_kernel, dim3(max_splits, G, T), dim3(DC_WARPS * 32), smem, stream, 1, a);
  if (rc) return say(err, err_len, rc, "the kernel launch failed (%lld)", rc);
  return 0;
}

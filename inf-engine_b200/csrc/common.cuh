// Shared helpers of the engine's CUDA kernels (sm_100a).
//
// Every launcher is an extern "C" function over raw device pointers and a
// stream, so the library carries no framework headers and builds in seconds.
// A launcher returns 0, a positive cudaError_t from the launch, or a negative
// code of this file when it refuses its arguments.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <tuple>
#include <utility>

#define IE_OK 0
#define IE_BAD_DTYPE -1
#define IE_BAD_SIZE -2
#define IE_BAD_ALIGN -3

// dtype codes used across the C interface
#define IE_F32 0
#define IE_BF16 1

typedef __nv_bfloat16 bf16;

// A checks build (-DIE_CHECKS=1; `kernels.enable_checks()`): every page id, cache slot and token id that a kernel reads
// from memory is compared with limits that the host has set (ie_check_limits_<unit>).  A value out of range is
// recorded in a device word of the unit (the first one with its code, value and limit, and a count of all) and
// replaced by a safe one (no page, no slot, token 0): nothing is read or written out of bounds and nothing traps;
// the host reads the word (ie_check_read_<unit>) when the step is done.  Without the switch the macros are the value.
// Codes: 1 page id, 2 cache slot, 3 token id.
#ifdef IE_CHECKS
static __device__ int g_check_word[4];
static __device__ int g_check_limit[3] = {0x7fffffff, 0x7fffffff, 0x7fffffff};   // pages, slots, vocabulary
__device__ __forceinline__ void ie_check_record(int code, int value, int limit) {
  if (atomicCAS(&g_check_word[0], 0, code) == 0) {
    g_check_word[1] = value;
    g_check_word[2] = limit;
  }
  atomicAdd(&g_check_word[3], 1);
}
__device__ __forceinline__ int ie_checked(int v, int lo, int code, int safe) {
  const int hi = g_check_limit[code - 1];
  if (v >= lo && v < hi) return v;
  ie_check_record(code, v, hi);
  return safe;
}
#define IE_PAGE(v) ie_checked((v), -1, 1, -1)     /* -1: a page that is not held */
#define IE_SLOT(v) ie_checked((v), -1, 2, -1)     /* -1: nothing is stored */
#define IE_TOKEN(v) ie_checked((v), 0, 3, 0)
#define IE_CHECK_API(unit)                                                                              \
  extern "C" int ie_check_limits_##unit(int pages, int slots, int vocab) {                              \
    const int lim[3] = {pages, slots, vocab};                                                           \
    return (int)cudaMemcpyToSymbol(g_check_limit, lim, sizeof(lim));                                    \
  }                                                                                                     \
  extern "C" int ie_check_read_##unit(int* out4) {                                                      \
    const int zero[4] = {0, 0, 0, 0};                                                                   \
    cudaError_t e = cudaMemcpyFromSymbol(out4, g_check_word, sizeof(zero));                             \
    if (e == cudaSuccess && out4[3]) e = cudaMemcpyToSymbol(g_check_word, zero, sizeof(zero));          \
    return (int)e;                                                                                      \
  }
#else
#define IE_PAGE(v) (v)
#define IE_SLOT(v) (v)
#define IE_TOKEN(v) (v)
#define IE_CHECK_API(unit)
#endif

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

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

// Sum over a block in a fixed order (warp trees, then the warps in order): the
// result does not depend on timing.  `scratch` holds at least 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < n_warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < n_warps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---------------------------------------------------- programmatic dependent launch
// Every kernel of this package is launched so that it may start while the kernel
// before it in the stream is still running (its blocks become resident once all
// blocks of the predecessor have called pdl_trigger or exited).  A kernel may
// read only data that no kernel writes (weights, tables, the step's metadata
// copied in before the step) until it has called pdl_wait, which returns when the
// predecessor has finished and its writes are visible; it writes nothing before
// that.  This hides launch latency and lets weight-streaming kernels fetch their
// first weights early.  Every block calls pdl_wait, so completion of a kernel
// implies completion of everything before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// -DIE_NO_PDL=1 builds a library whose launches do not carry the attribute (for comparisons; the package never sets it)
static inline bool pdl_enabled() {
#if defined(IE_NO_PDL) && IE_NO_PDL
  return false;
#else
  return true;
#endif
}

// cluster_x > 1: consecutive blocks along x form thread-block clusters of that size (grid.x a multiple of it)
static inline int launch_raw(const void* kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             void** args, int cluster_x = 1) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelExC(&cfg, kernel, args);
}

template <typename Tuple, size_t... I>
static inline void tuple_pointers(Tuple& t, void** out, std::index_sequence<I...>) {
  ((out[I] = (void*)&std::get<I>(t)), ...);
}

// launch_k(kernel, grid, block, smem, stream, args...): arguments are converted to the kernel's parameter types
template <typename... KArgs, typename... Args>
static inline int launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args... args) {
  static_assert(sizeof...(KArgs) == sizeof...(Args), "kernel argument count");
  std::tuple<KArgs...> vals{static_cast<KArgs>(args)...};
  void* ptrs[sizeof...(KArgs) ? sizeof...(KArgs) : 1];
  tuple_pointers(vals, ptrs, std::index_sequence_for<KArgs...>{});
  return launch_raw((const void*)kernel, grid, block, smem, stream, ptrs);
}

// the same with clusters of cluster_x blocks along x
template <typename... KArgs, typename... Args>
static inline int launch_k_cluster(void (*kernel)(KArgs...), int cluster_x, dim3 grid, dim3 block, size_t smem,
                                   cudaStream_t stream, Args... args) {
  static_assert(sizeof...(KArgs) == sizeof...(Args), "kernel argument count");
  std::tuple<KArgs...> vals{static_cast<KArgs>(args)...};
  void* ptrs[sizeof...(KArgs) ? sizeof...(KArgs) : 1];
  tuple_pointers(vals, ptrs, std::index_sequence_for<KArgs...>{});
  return launch_raw((const void*)kernel, grid, block, smem, stream, ptrs, cluster_x);
}

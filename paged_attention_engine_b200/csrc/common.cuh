// Shared helpers of the kernel files: element types, error reporting, launch checks.
//
// Every entry point is `extern "C"`, takes raw device pointers and sizes, launches on the
// stream it is given and returns 0, or a non-zero code after storing a message that
// `pae_last_error()` of the same library returns. A size that a kernel cannot take is
// refused with such a message before anything is launched; no entry point falls back to
// another device or to the host.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <utility>

namespace pae {

enum DType : int { kF32 = 0, kBF16 = 1 };

inline char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

inline int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(error_buffer(), 512, format, args);
  va_end(args);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(100, "%s: %s", what, cudaGetErrorString(err));
  return 0;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One rotation of a pair (engine/model.py:155-161): lo' = lo c - hi s, hi' = hi c + lo s, each
// product and each sum rounded on its own. Several kernels rotate (stand-alone, inside the sum
// of a split product, inside a product's epilogue) and must give the same bits; left to the
// compiler, one kernel would fuse a multiply into the add and another would not.
__device__ __forceinline__ void rotate_pair(float& lo, float& hi, float c, float s) {
  const float new_lo = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s));
  const float new_hi = __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s));
  lo = new_lo;
  hi = new_hi;
}

// ---------------------------------------------------------------------------------------
// The checked build (-DPAE_BOUNDS, `PAE_BOUNDS=1` for kernels/build.py): every slot, block-table
// index and page id that a kernel takes from the step's integer arrays is compared with what
// the cache holds before it becomes an address. A value out of range sets the device's error
// word (101: a slot beyond the pool; 102: a block-table index beyond the table's width; 103: a
// page id that is negative or beyond the pool) and the access is not made: a write is
// skipped, a read goes to page 0 instead. Nothing traps; the host reads the word like that of a
// wait that gave up. In the ordinary build the helpers below are the identity and cost nothing.
// The limits reach a library through `pae_set_bounds(pages, error word)`.
// ---------------------------------------------------------------------------------------
#ifdef PAE_BOUNDS
struct Bounds {
  long long pages;
  int* error;
};
__device__ Bounds g_bounds = {0, nullptr};
__device__ __forceinline__ void bounds_violation(int code) {
  if (g_bounds.error != nullptr) atomicCAS(g_bounds.error, 0, code);
}
#endif

__device__ __forceinline__ bool slot_in_pool(int slot, int page_size) {
#ifdef PAE_BOUNDS
  if (g_bounds.pages > 0 && (slot < 0 || (long long)(slot / page_size) >= g_bounds.pages)) {
    bounds_violation(101);
    return false;
  }
#endif
  return true;
}

__device__ __forceinline__ int checked_table_index(int index, int width) {
#ifdef PAE_BOUNDS
  if (index < 0 || index >= width) {
    bounds_violation(102);
    return 0;
  }
#endif
  return index;
}

__device__ __forceinline__ int checked_page(int page) {
#ifdef PAE_BOUNDS
  if (g_bounds.pages > 0 && (page < 0 || (long long)page >= g_bounds.pages)) {
    bounds_violation(103);
    return 0;
  }
#endif
  return page;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Programmatic dependent launch. Every kernel of these libraries starts with
// `dependent_launch_prologue()` (for the tensor-core product: after its set-up that touches no
// global memory) and is launched with `launch_kernel`, which marks it as allowed to start
// while the kernel before it in the stream is still finishing. The prologue first lets the
// NEXT kernel begin to launch, then waits until the kernel BEFORE has completed and its
// writes are visible; nothing of global memory is read or written before that wait. So the
// order of all memory effects is that of a plain stream, and only launch latencies and
// prologues overlap. A step of decoding is several hundred small kernels; this is worth
// about a third of its time. PAE_PDL=0 in the environment turns it off.
//
// A few kernels do read before the wait. The rule they keep: only memory that was last written
// before the kernel BEFORE this one was launched, which is the only memory certain to be
// complete at that point whatever the stream did between the two launches. The products and
// the fused norm read their weights (written when the model was loaded); decode attention reads the step's
// integers and the keys and values of earlier tokens (written in earlier steps, and by the
// copy that opens the step, which many kernels follow before the first attention); the merge
// follows the sliced kernel of the same call. Everything else before a wait is a prefetch hint.
__device__ __forceinline__ void dependent_launch_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void dependent_launch_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dependent_launch_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool dependent_launch_enabled() {
  static const bool enabled = [] {
    const char* v = std::getenv("PAE_PDL");
    return v == nullptr || std::atoi(v) != 0;
  }();
  return enabled;
}

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, KArgs(std::forward<Args>(args))...);   // errors surface in check_launch
}

// The same for a kernel whose blocks form clusters of `cluster_x` along x (distributed shared memory).
template <typename... KArgs, typename... Args>
inline void launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster_x;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&config, kernel, KArgs(std::forward<Args>(args))...);
}

}  // namespace pae

#define PAE_EXPORT extern "C" __attribute__((visibility("default")))

// Each library exports its own message getter (and, in the checked build, the setter of its limits).
#ifdef PAE_BOUNDS
#define PAE_DEFINE_LAST_ERROR()                                                                     \
  PAE_EXPORT const char* pae_last_error() { return pae::error_buffer(); }                           \
  PAE_EXPORT int pae_set_bounds(long long pages, int* error) {                                      \
    pae::Bounds b{pages, error};                                                                    \
    cudaError_t err = cudaMemcpyToSymbol(pae::g_bounds, &b, sizeof(b));                             \
    if (err != cudaSuccess) return pae::fail(100, "set_bounds: %s", cudaGetErrorString(err));       \
    return 0;                                                                                       \
  }
#else
#define PAE_DEFINE_LAST_ERROR() \
  PAE_EXPORT const char* pae_last_error() { return pae::error_buffer(); }
#endif

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

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace pae

#define PAE_EXPORT extern "C" __attribute__((visibility("default")))

// Each library exports its own message getter.
#define PAE_DEFINE_LAST_ERROR() \
  PAE_EXPORT const char* pae_last_error() { return pae::error_buffer(); }

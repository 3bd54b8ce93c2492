// The allocation-free variant of decode attention declared in attention_decode_noalloc.h:
// the same kernels as pae_paged_attention_decode (attention_mma.cuh), with the per-slice
// partial results in a fixed array of this library instead of a buffer from the caller.
#include "attention_decode_noalloc.h"

#include <mutex>

#include "attention_mma.cuh"

using namespace pae;
using namespace pae_attention;

// The scratch itself. In host code this name is only a handle for the runtime, not a
// device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float noalloc_scratch[PAE_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
float* scratch_of_device[MAX_DEVICES] = {nullptr};
std::mutex setup_mutex;

// The device address of the array on the current device; looked up once per device.
int scratch_address(float** address) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(100, "paged_attention_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(err));
  if (device < 0 || device >= MAX_DEVICES) return fail(3, "paged_attention_decode_noalloc: device %d is beyond the %d this library keeps track of", device, MAX_DEVICES);
  std::lock_guard<std::mutex> guard(setup_mutex);
  if (scratch_of_device[device] == nullptr) {
    float* ptr = nullptr;
    err = cudaGetSymbolAddress((void**)&ptr, noalloc_scratch);
    if (err != cudaSuccess || ptr == nullptr)
      return fail(100, "paged_attention_decode_noalloc: cudaGetSymbolAddress on device %d: %s", device, cudaGetErrorString(err));
    scratch_of_device[device] = ptr;
  }
  *address = scratch_of_device[device];
  return 0;
}

}  // namespace

PAE_EXPORT long long pae_noalloc_scratch_capacity(void) { return PAE_NOALLOC_SCRATCH_FLOATS; }

PAE_EXPORT int pae_paged_attention_decode_noalloc(void* out, const void* qkv, const void* keys, const void* values,
                                                  const int* block_table, int table_width, const int* q_start,
                                                  const int* kv_len, int seqs, int heads, int kv_heads, int d,
                                                  int page_size, float scale, int window, int slice_keys, int max_slices,
                                                  void* stream) {
  if (seqs == 0) return 0;
  if (seqs < 0 || heads < 1 || d < 1 || max_slices < 1)
    return fail(2, "paged_attention_decode_noalloc: %d requests, %d heads of %d, %d slices", seqs, heads, d, max_slices);
  const long long needed = decode_scratch_floats(seqs, heads, d, max_slices);
  if (needed > PAE_NOALLOC_SCRATCH_FLOATS)
    return fail(4,
                "paged_attention_decode_noalloc: %d requests x %d heads x %d slices need %lld floats of scratch, the library "
                "holds %d; use fewer or longer slices, or pae_paged_attention_decode with a buffer of your own",
                seqs, heads, max_slices, needed, PAE_NOALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  if (int err = scratch_address(&scratch)) return err;
  return decode_with_scratch(out, qkv, keys, values, block_table, table_width, q_start, kv_len, seqs, heads, kv_heads, d,
                             page_size, scale, window, slice_keys, max_slices, scratch, (cudaStream_t)stream);
}

PAE_DEFINE_LAST_ERROR()

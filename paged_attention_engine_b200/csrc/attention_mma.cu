// Exported entry points of the tensor-core attention kernels of attention_mma.cuh.
#include "attention_mma.cuh"

using namespace pae;
using namespace pae_attention;

// 1 when these kernels take the sizes (the caller then need not try and catch a refusal).
PAE_EXPORT int pae_attention_mma_supports(int heads, int kv_heads, int d, int page_size) {
  return (d == 32 || d == 64 || d == 128) && page_size >= 16 && page_size % 16 == 0 && kv_heads >= 1 &&
         heads % kv_heads == 0 && heads / kv_heads <= 16;
}

// How many slices a block of the decode kernel takes.
PAE_EXPORT int pae_decode_slices_per_block() { return SLICE_WARPS; }

// How many blocks of the decode kernel the device holds at one time: the
// slicing aims at one such wave, since a second, partly filled one costs as much as a full one.
PAE_EXPORT int pae_decode_blocks_per_wave(int d) {
  static int cached[3] = {0, 0, 0};
  const int which = d == 32 ? 0 : (d == 64 ? 1 : 2);
  if (cached[which] == 0) {
    int device = 0, sms = 148, per_sm = 0;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const size_t bytes = slices_smem_bytes(d == 32 ? 32 : (d == 64 ? 64 : 128));
    cudaError_t err;
    if (d == 32) {
      allow_smem(decode_slices_kernel<32>, bytes, "paged_attention_decode");
      err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_slices_kernel<32>, SLICE_WARPS * 32, bytes);
    } else if (d == 64) {
      allow_smem(decode_slices_kernel<64>, bytes, "paged_attention_decode");
      err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_slices_kernel<64>, SLICE_WARPS * 32, bytes);
    } else {
      allow_smem(decode_slices_kernel<128>, bytes, "paged_attention_decode");
      err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_slices_kernel<128>, SLICE_WARPS * 32, bytes);
    }
    cached[which] = (err == cudaSuccess && per_sm > 0 ? per_sm : 1) * sms;
  }
  return cached[which];
}

// Floats of scratch that `pae_paged_attention_decode` needs for `seqs` requests and `max_slices` slices.
PAE_EXPORT long long pae_decode_scratch_floats(int seqs, int heads, int d, int max_slices) {
  return decode_scratch_floats(seqs, heads, d, max_slices);
}

// Requests that bring exactly one token: out[token, head, :] over keys [0, kv_len) (or the
// last `window`). Requests with more tokens are skipped. `scratch` holds
// pae_decode_scratch_floats(...) floats; `slice_keys` is a multiple of 16 and
// max_slices * slice_keys covers the longest request.
PAE_EXPORT int pae_paged_attention_decode(void* out, const void* qkv, const void* keys, const void* values,
                                          const int* block_table, int table_width, const int* q_start,
                                          const int* kv_len, int seqs, int heads, int kv_heads, int d, int page_size,
                                          float scale, int window, int slice_keys, int max_slices, float* scratch,
                                          void* stream) {
  return decode_with_scratch(out, qkv, keys, values, block_table, table_width, q_start, kv_len, seqs, heads, kv_heads, d,
                             page_size, scale, window, slice_keys, max_slices, scratch, (cudaStream_t)stream);
}

// Requests that bring several tokens (and, unless skip_single, those that bring one); with
// `work_index` (device, `work_count` entries) only the requests it lists get blocks.
PAE_EXPORT int pae_paged_attention_prefill(void* out, const void* qkv, const void* keys, const void* values,
                                           const int* block_table, int table_width, const int* q_start,
                                           const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads,
                                           int kv_heads, int d, int page_size, float scale, int window,
                                           int skip_single, const int* work_index, int work_count, void* stream) {
  if (seqs == 0 || max_q_len == 0) return 0;
  if (int err = check_sizes("paged_attention_prefill", heads, kv_heads, d, page_size, seqs)) return err;
  if (work_index != nullptr && (work_count < 1 || work_count > seqs))
    return fail(2, "paged_attention_prefill: a list of %d requests to work on, of %d", work_count, seqs);
  PrefillParams p{};
  p.out = (__nv_bfloat16*)out;
  p.qkv = (const __nv_bfloat16*)qkv;
  p.keys = (const __nv_bfloat16*)keys;
  p.values = (const __nv_bfloat16*)values;
  p.block_table = block_table;
  p.q_start = q_start;
  p.q_pos0 = q_pos0;
  p.kv_len = kv_len;
  p.table_width = table_width;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.page_size = page_size;
  p.window = window;
  p.skip_single = skip_single;
  p.work_index = work_index;
  p.scale_log2 = scale * LOG2E;
  cudaStream_t s = (cudaStream_t)stream;
  const int covered = work_index != nullptr ? work_count : seqs;       // grid z: the listed requests, or all
  if (d == 32) return launch_prefill<32>(p, covered, max_q_len, s);
  if (d == 64) return launch_prefill<64>(p, covered, max_q_len, s);
  return launch_prefill<128>(p, covered, max_q_len, s);
}

PAE_DEFINE_LAST_ERROR()

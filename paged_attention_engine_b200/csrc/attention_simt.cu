// Attention over the paged cache on the CUDA cores, for every size: any head size that
// is a multiple of 8 up to 256, any number of heads and kv heads, any page size, with
// or without a window, portions of prompts and single decoded tokens in one launch.
// It is the attention of the true 32-bit path, and in the bfloat16 path it takes what
// the tensor-core kernels refuse.
//
// The reference gathers each request's whole key/value history into a padded buffer,
// repeats kv heads for the query heads and calls a library with a boolean mask
// (engine/attention.py:597-624,46-74). Here a block owns 16 consecutive query tokens of
// one request and one query head, walks that request's pages in place through its block
// table, 32 keys at a time, and keeps a running softmax (max, sum) in float32. The rule
// of engine/attention.py:581-586 is evaluated per score: key j is seen by the query at
// position p when j <= p and j < kv_len, and p - j < window when the layer has one.
// Query head h reads kv head h / (heads / kv_heads).
//
// A query's result depends only on its own keys: the tile a token falls in changes the
// order in which its keys are folded in by at most the tile start, never the values.
#include "common.cuh"

#include <cfloat>

using namespace pae;

namespace {

constexpr int BQ = 16;      // query tokens per block
constexpr int BKEYS = 32;   // keys per iteration
constexpr int THREADS = 128;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS) paged_attention_simt_kernel(
    T* __restrict__ out, const T* __restrict__ qkv, const T* __restrict__ keys, const T* __restrict__ values,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ q_start,
    const int* __restrict__ q_pos0, const int* __restrict__ kv_len, int heads, int kv_heads, int d, int page_size,
    float scale, int window) {
  dependent_launch_prologue();
  extern __shared__ float smem[];
  const int b = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int first_token = q_start[b];
  const int q_count = q_start[b + 1] - first_token;
  if (tile * BQ >= q_count) return;
  const int p0 = q_pos0[b] + tile * BQ;                // position of the tile's first query
  const int rows = min(BQ, q_count - tile * BQ);
  const int kv_end = min(kv_len[b], p0 + rows);         // keys past the last query are never seen
  const int kv_begin = window > 0 ? max(0, p0 - window + 1) : 0;
  const int g = h / (heads / kv_heads);
  const int qkv_width = (heads + 2 * kv_heads) * d;

  const int dpad = d + 1;
  float* qs = smem;                        // [BQ][d + 1]
  float* ks = qs + BQ * dpad;              // [BKEYS][d + 1]
  float* vs = ks + BKEYS * dpad;           // [BKEYS][d]
  float* ps = vs + BKEYS * d;              // [BQ][BKEYS + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid >> 3;                  // query row of this thread, 0..15
  const int cg = tid & 7;                  // column group: keys cg + 8 i, dims cg + 8 i

  for (int i = tid; i < BQ * d; i += THREADS) {
    const int row = i / d, k = i - row * d;
    qs[row * dpad + k] = row < rows ? to_float(qkv[(size_t)(first_token + tile * BQ + row) * qkv_width + h * d + k]) : 0.f;
  }

  float acc[MAX_D / 8];
#pragma unroll
  for (int i = 0; i < MAX_D / 8; ++i) acc[i] = 0.f;
  float row_max = -FLT_MAX, row_sum = 0.f;
  const int my_pos = p0 + r;
  const int nd = d >> 3;
  const int* table = block_table + (size_t)b * table_width;

  for (int base = kv_begin; base < kv_end; base += BKEYS) {
    __syncthreads();   // the previous iteration's reads of ks, vs, ps are done (and qs is written)
    // Each warp brings 8 of the 32 keys; lanes run along the head dimension.
    for (int c = warp; c < BKEYS; c += THREADS / 32) {
      const int j = base + c;
      if (j < kv_end) {
        const int page = checked_page(table[checked_table_index(j / page_size, table_width)]);
        const size_t at = (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * d;
        for (int k = lane; k < d; k += 32) {
          ks[c * dpad + k] = to_float(keys[at + k]);
          vs[c * d + k] = to_float(values[at + k]);
        }
      } else {
        for (int k = lane; k < d; k += 32) {
          ks[c * dpad + k] = 0.f;
          vs[c * d + k] = 0.f;
        }
      }
    }
    __syncthreads();

    float s[BKEYS / 8];
    float tile_max = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < BKEYS / 8; ++i) {
      const int c = cg + 8 * i;
      const int j = base + c;
      float dot = 0.f;
      for (int k = 0; k < d; ++k) dot = fmaf(qs[r * dpad + k], ks[c * dpad + k], dot);
      const bool seen = r < rows && j < kv_end && j <= my_pos && (window <= 0 || my_pos - j < window);
      s[i] = seen ? dot * scale : -FLT_MAX;
      tile_max = fmaxf(tile_max, s[i]);
    }
    // The 8 threads of a row are 8 neighbouring lanes.
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
    const float new_max = fmaxf(row_max, tile_max);
    const float rescale = (row_max == -FLT_MAX) ? 0.f : expf(row_max - new_max);
    float tile_sum = 0.f;
#pragma unroll
    for (int i = 0; i < BKEYS / 8; ++i) {
      const float p = (s[i] == -FLT_MAX) ? 0.f : expf(s[i] - new_max);
      ps[r * (BKEYS + 1) + cg + 8 * i] = p;
      tile_sum += p;
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, o);
    row_sum = row_sum * rescale + tile_sum;
    row_max = new_max;
    __syncwarp();   // ps of a row is written and read by the same 8 lanes of one warp
#pragma unroll
    for (int i = 0; i < MAX_D / 8; ++i) {
      if (i < nd) {
        float v = acc[i] * rescale;
        const int dim = cg + 8 * i;
        for (int c = 0; c < BKEYS; ++c) v = fmaf(ps[r * (BKEYS + 1) + c], vs[c * d + dim], v);
        acc[i] = v;
      }
    }
  }

  if (r < rows) {
    const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
    T* to = out + ((size_t)(first_token + tile * BQ + r) * heads + h) * d;
#pragma unroll
    for (int i = 0; i < MAX_D / 8; ++i)
      if (i < nd) to[cg + 8 * i] = from_float<T>(acc[i] * inv);
  }
}

size_t smem_bytes(int d) { return sizeof(float) * (size_t)(BQ * (d + 1) + BKEYS * (d + 1) + BKEYS * d + BQ * (BKEYS + 1)); }

template <typename T>
int launch(void* out, const void* qkv, const void* keys, const void* values, const int* block_table, int table_width,
           const int* q_start, const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads, int kv_heads,
           int d, int page_size, float scale, int window, cudaStream_t s) {
  const size_t bytes = smem_bytes(d);
  auto kernel = paged_attention_simt_kernel<T>;
  static bool raised = false;   // per element type: the limit is raised once, to the most any head size needs
  if (bytes > 48 * 1024 && !raised) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(MAX_D));
    if (err != cudaSuccess) return fail(100, "paged_attention_simt: %s", cudaGetErrorString(err));
    raised = true;
  }
  dim3 grid((max_q_len + BQ - 1) / BQ, heads, seqs);
  launch_kernel(kernel, grid, THREADS, bytes, s, (T*)out, (const T*)qkv, (const T*)keys, (const T*)values, block_table,
                                      table_width, q_start, q_pos0, kv_len, heads, kv_heads, d, page_size, scale, window);
  return check_launch("paged_attention_simt");
}

}  // namespace

// out [tokens, heads, d]; qkv [tokens, heads + 2 kv_heads, d] (queries are read from it);
// keys, values [pages, kv_heads, page_size, d]; block_table [seqs, table_width].
PAE_EXPORT int pae_paged_attention_simt(void* out, const void* qkv, const void* keys, const void* values,
                                        const int* block_table, int table_width, const int* q_start,
                                        const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads,
                                        int kv_heads, int d, int page_size, float scale, int window, int dtype,
                                        void* stream) {
  if (seqs == 0 || max_q_len == 0) return 0;
  if (d % 8 || d > MAX_D || d < 8) return fail(2, "paged_attention_simt: head_dim %d is not a multiple of 8 in [8, %d]", d, MAX_D);
  if (kv_heads < 1 || heads % kv_heads) return fail(2, "paged_attention_simt: %d heads over %d kv heads", heads, kv_heads);
  if (heads > 65535 || seqs > 65535) return fail(3, "paged_attention_simt: %d heads x %d requests exceed one launch", heads, seqs);
  if (page_size < 1) return fail(2, "paged_attention_simt: page size %d", page_size);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    return launch<float>(out, qkv, keys, values, block_table, table_width, q_start, q_pos0, kv_len, seqs, max_q_len, heads, kv_heads, d, page_size, scale, window, s);
  if (dtype == kBF16)
    return launch<__nv_bfloat16>(out, qkv, keys, values, block_table, table_width, q_start, q_pos0, kv_len, seqs, max_q_len, heads, kv_heads, d, page_size, scale, window, s);
  return fail(1, "paged_attention_simt: unknown dtype %d", dtype);
}

PAE_DEFINE_LAST_ERROR()

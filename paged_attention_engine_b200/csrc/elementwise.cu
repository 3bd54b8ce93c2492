// Memory-bound kernels of the step: embedding gather, RMSNorm, the rotary table, the
// rotation of q and k fused with the write of k and v into their pages, SiLU x up, and
// the row gather before the head. One template over the element type serves the true
// 32-bit path and the bfloat16 path; all arithmetic is float32 and each result is
// rounded once.
#include "common.cuh"

using namespace pae;

// ------------------------------------------------------------------------------------
// Row gather: out[r, :] = table[index[r], :]. An index outside [0, rows) yields zeros.
// Serves the token embedding (engine/model.py:401 of the reference) and the gather of
// the rows whose logits are wanted (engine/model.py:453-454).
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ table,
                                   const int* __restrict__ index, int rows, int width) {
  const int r = blockIdx.x;
  const int src = index[r];
  const bool ok = src >= 0 && src < rows;
  const T* from = table + (size_t)(ok ? src : 0) * width;
  T* to = out + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = ok ? from[i] : from_float<T>(0.f);
}

PAE_EXPORT int pae_gather_rows(void* out, const void* table, const int* index, int n, int rows, int width,
                               int dtype, void* stream) {
  if (n == 0) return 0;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    gather_rows_kernel<float><<<n, threads, 0, s>>>((float*)out, (const float*)table, index, rows, width);
  else if (dtype == kBF16)
    gather_rows_kernel<__nv_bfloat16><<<n, threads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)table, index, rows, width);
  else
    return fail(1, "gather_rows: unknown dtype %d", dtype);
  return check_launch("gather_rows");
}

// ------------------------------------------------------------------------------------
// RMSNorm (engine/model.py:117-123): y = w * x * rsqrt(mean(x^2) + eps), statistics and
// scaling in float32, weight in float32, one rounding at the end. One block per row;
// the order of the sum depends on the width only, never on the batch.
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void rms_norm_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ weight,
                                int width, float eps) {
  __shared__ float partial[32];
  const T* row = x + (size_t)blockIdx.x * width;
  float sum = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(row[i]);
    sum += v * v;
  }
  sum = warp_sum(sum);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float v = lane < warps ? partial[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) partial[0] = rsqrtf(v / (float)width + eps);
  }
  __syncthreads();
  const float scale = partial[0];
  T* to = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from_float<T>(to_float(row[i]) * scale * weight[i]);
}

PAE_EXPORT int pae_rms_norm(void* out, const void* x, const float* weight, int rows, int width, float eps,
                            int dtype, void* stream) {
  if (rows == 0) return 0;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : (width >= 128 ? 128 : 32));
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    rms_norm_kernel<float><<<rows, threads, 0, s>>>((float*)out, (const float*)x, weight, width, eps);
  else if (dtype == kBF16)
    rms_norm_kernel<__nv_bfloat16><<<rows, threads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, weight, width, eps);
  else
    return fail(1, "rms_norm: unknown dtype %d", dtype);
  return check_launch("rms_norm");
}

// ------------------------------------------------------------------------------------
// Rotary table (engine/model.py:138-152): angle = float(position) * inv_freq[i] as one
// float32 product, then its cosine (first half of the row) and sine (second half).
// ------------------------------------------------------------------------------------
__global__ void rotary_table_kernel(float* __restrict__ table, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int tokens, int half) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * half) return;
  const int t = i / half, f = i - t * half;
  const float angle = (float)positions[t] * inv_freq[f];
  float s, c;
  sincosf(angle, &s, &c);
  table[(size_t)t * 2 * half + f] = c;
  table[(size_t)t * 2 * half + half + f] = s;
}

PAE_EXPORT int pae_rotary_table(float* table, const int* positions, const float* inv_freq, int tokens, int half,
                                void* stream) {
  const long long n = (long long)tokens * half;
  if (n == 0) return 0;
  rotary_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(table, positions, inv_freq, tokens, half);
  return check_launch("rotary_table");
}

// ------------------------------------------------------------------------------------
// Rotation of q and k (pairs (j, j + d/2): engine/model.py:126-129,155-161) in place in
// the fused projection's output [tokens, heads + 2 kv_heads, d], and the write of the
// rotated k and of v into the pages: slot = page * page_size + offset selects
// keys[page, kv_head, offset, :] (the reference's only address translation,
// engine/attention.py:374-385, scatter at :613-616). `table` may be null (no rotation);
// `slots` may be null (an entry that reads another entry's cache writes nothing).
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void rotary_qk_cache_write_kernel(T* __restrict__ qkv, const float* __restrict__ table,
                                             const int* __restrict__ slots, T* __restrict__ keys,
                                             T* __restrict__ values, int tokens, int heads, int kv_heads, int d,
                                             int page_size) {
  const int half = d >> 1;
  const int per_token = (heads + 2 * kv_heads) * half;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * per_token) return;
  const int t = (int)(i / per_token);
  const int rest = (int)(i - (long long)t * per_token);
  const int head = rest / half, f = rest - head * half;
  T* at = qkv + ((size_t)t * (heads + 2 * kv_heads) + head) * d;
  float lo = to_float(at[f]), hi = to_float(at[f + half]);
  if (head < heads + kv_heads && table != nullptr) {
    const float c = table[(size_t)t * d + f], s = table[(size_t)t * d + half + f];
    const float new_lo = lo * c - hi * s;
    const float new_hi = hi * c + lo * s;
    lo = new_lo;
    hi = new_hi;
    at[f] = from_float<T>(lo);
    at[f + half] = from_float<T>(hi);
  }
  if (head >= heads && slots != nullptr) {
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, offset = slot - page * page_size;
    const bool is_key = head < heads + kv_heads;
    const int kv_head = is_key ? head - heads : head - heads - kv_heads;
    T* to = (is_key ? keys : values) + (((size_t)page * kv_heads + kv_head) * page_size + offset) * d;
    to[f] = from_float<T>(lo);
    to[f + half] = from_float<T>(hi);
  }
}

PAE_EXPORT int pae_rotary_qk_cache_write(void* qkv, const float* table, const int* slots, void* keys, void* values,
                                         int tokens, int heads, int kv_heads, int d, int page_size, int dtype,
                                         void* stream) {
  if (d % 2) return fail(2, "rotary_qk_cache_write: head_dim %d is odd", d);
  const long long n = (long long)tokens * (heads + 2 * kv_heads) * (d / 2);
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    rotary_qk_cache_write_kernel<float><<<blocks, 256, 0, s>>>((float*)qkv, table, slots, (float*)keys, (float*)values, tokens, heads, kv_heads, d, page_size);
  else if (dtype == kBF16)
    rotary_qk_cache_write_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)qkv, table, slots, (__nv_bfloat16*)keys, (__nv_bfloat16*)values, tokens, heads, kv_heads, d, page_size);
  else
    return fail(1, "rotary_qk_cache_write: unknown dtype %d", dtype);
  return check_launch("rotary_qk_cache_write");
}

// ------------------------------------------------------------------------------------
// SwiGLU's middle (engine/model.py:317-320): out[t, i] = silu(gate[t, i]) * up[t, i]
// where a row of the input holds the gate in [0, I) and the up projection in [I, 2I).
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, long long total, int inter) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / inter;
  const int c = (int)(i - t * inter);
  const float g = to_float(gate_up[t * 2 * inter + c]);
  const float u = to_float(gate_up[t * 2 * inter + inter + c]);
  out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

PAE_EXPORT int pae_silu_mul(void* out, const void* gate_up, int tokens, int inter, int dtype, void* stream) {
  const long long n = (long long)tokens * inter;
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    silu_mul_kernel<float><<<blocks, 256, 0, s>>>((float*)out, (const float*)gate_up, n, inter);
  else if (dtype == kBF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, n, inter);
  else
    return fail(1, "silu_mul: unknown dtype %d", dtype);
  return check_launch("silu_mul");
}

PAE_DEFINE_LAST_ERROR()

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
  dependent_launch_prologue();
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
    launch_kernel(gather_rows_kernel<float>, n, threads, 0, s, (float*)out, (const float*)table, index, rows, width);
  else if (dtype == kBF16)
    launch_kernel(gather_rows_kernel<__nv_bfloat16>, n, threads, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)table, index, rows, width);
  else
    return fail(1, "gather_rows: unknown dtype %d", dtype);
  return check_launch("gather_rows");
}

// ------------------------------------------------------------------------------------
// Token embedding with feedback. A negative token id stands for "the token this request
// sampled in the step before", which is still on the device: the kernel reads it from
// last_token[state_slot[seq_index[t]]]. `scatter_tokens` is what puts it there after
// sampling. Together they let the host plan the next step while this one runs; the
// reference reads every sampled token back before it goes on (engine/scheduler.py:610).
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_feedback_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                          const int* __restrict__ last_token, const int* __restrict__ state_slot,
                                          const int* __restrict__ seq_index, int rows, int width) {
  dependent_launch_prologue();
  const int t = blockIdx.x;
  int src = ids[t];
  if (src < 0) src = last_token[state_slot[seq_index[t]]];
  const bool ok = src >= 0 && src < rows;
  const T* from = table + (size_t)(ok ? src : 0) * width;
  T* to = out + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = ok ? from[i] : from_float<T>(0.f);
}

PAE_EXPORT int pae_embedding_feedback(void* out, const void* table, const int* ids, const int* last_token,
                                      const int* state_slot, const int* seq_index, int n, int rows, int width, int dtype,
                                      void* stream) {
  if (n == 0) return 0;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    launch_kernel(embedding_feedback_kernel<float>, n, threads, 0, s, (float*)out, (const float*)table, ids, last_token, state_slot, seq_index, rows, width);
  else if (dtype == kBF16)
    launch_kernel(embedding_feedback_kernel<__nv_bfloat16>, n, threads, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids, last_token, state_slot, seq_index, rows, width);
  else
    return fail(1, "embedding_feedback: unknown dtype %d", dtype);
  return check_launch("embedding_feedback");
}

// last_token[state_slot[seq_index[logit_rows[r]]]] = tokens[r] for every sampled row r.
__global__ void scatter_tokens_kernel(int* __restrict__ last_token, const int* __restrict__ tokens,
                                      const int* __restrict__ logit_rows, const int* __restrict__ seq_index,
                                      const int* __restrict__ state_slot, int n) {
  dependent_launch_prologue();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < n) last_token[state_slot[seq_index[logit_rows[r]]]] = tokens[r];
}

PAE_EXPORT int pae_scatter_tokens(int* last_token, const int* tokens, const int* logit_rows, const int* seq_index,
                                  const int* state_slot, int n, void* stream) {
  if (n == 0) return 0;
  launch_kernel(scatter_tokens_kernel, (n + 127) / 128, 128, 0, (cudaStream_t)stream, last_token, tokens, logit_rows, seq_index, state_slot, n);
  return check_launch("scatter_tokens");
}

// ------------------------------------------------------------------------------------
// RMSNorm (engine/model.py:117-123): y = w * x * rsqrt(mean(x^2) + eps), statistics and
// scaling in float32, weight in float32, one rounding at the end. One block per row;
// the order of the sum depends on the width only, never on the batch.
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void rms_norm_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ weight,
                                int width, float eps) {
  dependent_launch_prologue();
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

// The same for bfloat16 rows whose width is a multiple of 8: 16-byte loads and stores, the
// row kept in registers between the two passes. The sum runs over the same elements in
// another order than the scalar kernel's; the order depends on the width only.
template <int PER_THREAD>
__global__ void rms_norm_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                                       const float* __restrict__ weight, int width, float eps) {
  dependent_launch_prologue();
  __shared__ float partial[32];
  const int chunks = width >> 3;
  const uint4* row = (const uint4*)(x + (size_t)blockIdx.x * width);
  uint4 held[PER_THREAD];
  float4 w0[PER_THREAD], w1[PER_THREAD];        // the weight is asked for with the row, not after the sum
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER_THREAD; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < chunks) {
      held[j] = row[c];
      w0[j] = *(const float4*)(weight + c * 8);
      w1[j] = *(const float4*)(weight + c * 8 + 4);
    }
  }
#pragma unroll
  for (int j = 0; j < PER_THREAD; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < chunks) {
      const __nv_bfloat162* h = (const __nv_bfloat162*)&held[j];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        sum += f.x * f.x + f.y * f.y;
      }
    }
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
  uint4* to = (uint4*)(out + (size_t)blockIdx.x * width);
#pragma unroll
  for (int j = 0; j < PER_THREAD; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < chunks) {
      const __nv_bfloat162* h = (const __nv_bfloat162*)&held[j];
      uint4 packed;
      __nv_bfloat162* o = (__nv_bfloat162*)&packed;
      float2 f;
      f = __bfloat1622float2(h[0]); o[0] = __floats2bfloat162_rn(f.x * scale * w0[j].x, f.y * scale * w0[j].y);
      f = __bfloat1622float2(h[1]); o[1] = __floats2bfloat162_rn(f.x * scale * w0[j].z, f.y * scale * w0[j].w);
      f = __bfloat1622float2(h[2]); o[2] = __floats2bfloat162_rn(f.x * scale * w1[j].x, f.y * scale * w1[j].y);
      f = __bfloat1622float2(h[3]); o[3] = __floats2bfloat162_rn(f.x * scale * w1[j].z, f.y * scale * w1[j].w);
      to[c] = packed;
    }
  }
}

PAE_EXPORT int pae_rms_norm(void* out, const void* x, const float* weight, int rows, int width, float eps,
                            int dtype, void* stream) {
  if (rows == 0) return 0;
  if (dtype == kBF16 && width % 8 == 0 && width <= 8 * 4 * 256 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0 &&
      ((uintptr_t)weight & 15) == 0) {
    const int chunks = width / 8;
    const int block = chunks >= 256 ? 256 : ((chunks + 31) / 32) * 32;
    const int per_thread = (chunks + block - 1) / block;
    cudaStream_t vs = (cudaStream_t)stream;
    auto* o = (__nv_bfloat16*)out;
    auto* in = (const __nv_bfloat16*)x;
    if (per_thread == 1) launch_kernel(rms_norm_bf16x8_kernel<1>, rows, block, 0, vs, o, in, weight, width, eps);
    else if (per_thread == 2) launch_kernel(rms_norm_bf16x8_kernel<2>, rows, block, 0, vs, o, in, weight, width, eps);
    else launch_kernel(rms_norm_bf16x8_kernel<4>, rows, block, 0, vs, o, in, weight, width, eps);
    return check_launch("rms_norm");
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : (width >= 128 ? 128 : 32));
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    launch_kernel(rms_norm_kernel<float>, rows, threads, 0, s, (float*)out, (const float*)x, weight, width, eps);
  else if (dtype == kBF16)
    launch_kernel(rms_norm_kernel<__nv_bfloat16>, rows, threads, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, weight, width, eps);
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
  dependent_launch_prologue();
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
  launch_kernel(rotary_table_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, table, positions, inv_freq, tokens, half);
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
  dependent_launch_prologue();
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
    rotate_pair(lo, hi, c, s);
    at[f] = from_float<T>(lo);
    at[f + half] = from_float<T>(hi);
  }
  if (head >= heads && slots != nullptr) {
    const int slot = slots[t];
    if (slot < 0 || !slot_in_pool(slot, page_size)) return;
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
    launch_kernel(rotary_qk_cache_write_kernel<float>, blocks, 256, 0, s, (float*)qkv, table, slots, (float*)keys, (float*)values, tokens, heads, kv_heads, d, page_size);
  else if (dtype == kBF16)
    launch_kernel(rotary_qk_cache_write_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)qkv, table, slots, (__nv_bfloat16*)keys, (__nv_bfloat16*)values, tokens, heads, kv_heads, d, page_size);
  else
    return fail(1, "rotary_qk_cache_write: unknown dtype %d", dtype);
  return check_launch("rotary_qk_cache_write");
}

// ------------------------------------------------------------------------------------
// SwiGLU's middle (engine/model.py:317-320): out[t, i] = silu(gate[t, i]) * up[t, i]
// where a row of the input holds the gate in [0, I) and the up projection in [I, 2I).
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, long long total, int inter, int block) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / inter;
  const int c = (int)(i - t * inter);
  // block 0: gate in columns [0, I), up in [I, 2I); block b > 0: b gate columns, b up columns, and so on.
  const int gate_col = block > 0 ? (c / block) * 2 * block + c % block : c;
  const int up_col = block > 0 ? gate_col + block : inter + c;
  const float g = to_float(gate_up[t * 2 * inter + gate_col]);
  const float u = to_float(gate_up[t * 2 * inter + up_col]);
  out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// bfloat16 rows whose half-width is a multiple of 8: eight columns per thread, 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                       long long total_chunks, int inter) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_chunks) return;
  const int chunks = inter >> 3;
  const long long t = i / chunks;
  const int c = (int)(i - t * chunks);
  const uint4 g4 = *(const uint4*)(gate_up + t * 2 * inter + c * 8);
  const uint4 u4 = *(const uint4*)(gate_up + t * 2 * inter + inter + c * 8);
  const __nv_bfloat162* g = (const __nv_bfloat162*)&g4;
  const __nv_bfloat162* u = (const __nv_bfloat162*)&u4;
  uint4 packed;
  __nv_bfloat162* o = (__nv_bfloat162*)&packed;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 gf = __bfloat1622float2(g[e]), uf = __bfloat1622float2(u[e]);
    o[e] = __floats2bfloat162_rn(gf.x / (1.f + expf(-gf.x)) * uf.x, gf.y / (1.f + expf(-gf.y)) * uf.y);
  }
  *(uint4*)(out + t * inter + c * 8) = packed;
}

PAE_EXPORT int pae_silu_mul(void* out, const void* gate_up, int tokens, int inter, int block, int dtype, void* stream) {
  const long long n = (long long)tokens * inter;
  if (n == 0) return 0;
  if (block == 0 && dtype == kBF16 && inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    const long long chunks = n / 8;
    launch_kernel(silu_mul_bf16x8_kernel, (unsigned)((chunks + 255) / 256), 256, 0, (cudaStream_t)stream, 
        (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, chunks, inter);
    return check_launch("silu_mul");
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    launch_kernel(silu_mul_kernel<float>, blocks, 256, 0, s, (float*)out, (const float*)gate_up, n, inter, block);
  else if (dtype == kBF16)
    launch_kernel(silu_mul_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, n, inter, block);
  else
    return fail(1, "silu_mul: unknown dtype %d", dtype);
  return check_launch("silu_mul");
}

PAE_DEFINE_LAST_ERROR()

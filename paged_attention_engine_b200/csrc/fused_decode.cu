// Kernels that finish a split-K product inside the kernel that consumes it.
//
// In a step of few tokens the tcgen05 products leave float32 partial sums
// partial[split, token, n] (gemm_tcgen05.cu, SWAPPED form). Summing them is memory-trivial
// but a launch of its own; a decode step is bound by its number of launches, so the sum is
// folded into what comes next in the layer:
//
//   sum + residual -> new residual stream, and its RMSNorm        (after o_proj, down_proj)
//   sum -> SiLU(gate) x up                                        (after gate|up)
//   sum + bias -> rotation of q and k, page write of k and v      (after q|k|v)
//
// Every kernel sums the splits in their order, adds bias then residual in float32 and rounds
// the sum to the engine dtype before it goes on, exactly as the stand-alone reduction
// (pae_reduce_splits) followed by the stand-alone kernel does: the fused and the unfused
// paths give the same bits.
#include "common.cuh"

using namespace pae;

namespace {

// The sum of a column over the splits, in their order; the loads of twelve splits (then four,
// then one) are in flight together, so that a sum costs a trip or two to the L2, not one per split.
__device__ __forceinline__ float split_sum(const float* __restrict__ partial, int splits, size_t plane, size_t at) {
  float v = 0.f;
  int s = 0;
  for (; s + 12 <= splits; s += 12) {
    float p[12];
#pragma unroll
    for (int j = 0; j < 12; ++j) p[j] = partial[(size_t)(s + j) * plane + at];
#pragma unroll
    for (int j = 0; j < 12; ++j) v += p[j];
  }
  for (; s + 4 <= splits; s += 4) {
    float p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) p[j] = partial[(size_t)(s + j) * plane + at];
#pragma unroll
    for (int j = 0; j < 4; ++j) v += p[j];
  }
  for (; s < splits; ++s) v += partial[(size_t)s * plane + at];
  return v;
}

// value[row, :] = round(sum of splits + bias + residual); normed[row, :] = RMSNorm(value[row, :]) * weight.
template <typename T>
__global__ void __launch_bounds__(512) splitk_rms_norm_kernel(T* __restrict__ normed, T* __restrict__ value,
                                                              const float* __restrict__ partial, int splits,
                                                              const float* __restrict__ bias, const T* __restrict__ residual,
                                                              const float* __restrict__ weight, int rows, int width, float eps) {
  dependent_launch_prologue();
  extern __shared__ float row_values[];       // [width]: the rounded sums of this row
  __shared__ float reduce[32];
  const int row = blockIdx.x;
  const size_t plane = (size_t)rows * width;
  float squares = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const size_t at = (size_t)row * width + i;
    float v = split_sum(partial, splits, plane, at);
    if (bias != nullptr) v += bias[i];
    if (residual != nullptr) v += to_float(residual[at]);
    const T rounded = from_float<T>(v);
    value[at] = rounded;
    const float r = to_float(rounded);
    row_values[i] = r;
    squares += r * r;
  }
  squares = warp_sum(squares);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) reduce[warp] = squares;
  __syncthreads();
  if (warp == 0) {
    float v = lane < warps ? reduce[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) reduce[0] = rsqrtf(v / (float)width + eps);
  }
  __syncthreads();
  const float scale = reduce[0];
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    normed[(size_t)row * width + i] = from_float<T>(row_values[i] * scale * weight[i]);
}

// Four neighbouring values of T as floats, and back (16- or 8-byte accesses).
__device__ __forceinline__ void load4(const float* p, float* v) {
  const float4 t = *(const float4*)p;
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* v) {
  const uint2 t = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&t.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&t.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float* v) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* v) {
  uint2 t;
  *(__nv_bfloat162*)&t.x = __floats2bfloat162_rn(v[0], v[1]);
  *(__nv_bfloat162*)&t.y = __floats2bfloat162_rn(v[2], v[3]);
  *(uint2*)p = t;
}

// The same with four columns per thread (rows whose width is a multiple of 4 and tensors that
// start on 16 bytes): 16-byte loads of the partial sums, twelve splits in flight at a time. Sums
// run in the order of the splits, as above, so the rounded value is the same bits; the sum of
// squares adds four columns per thread first, which may differ from the scalar kernel in the
// last bit of the norm. A thread reads the norm's weight and the bias of its first four
// columns before anything else, and keeps the values of those columns in registers from the
// sum to the scaling, so nothing is read after the sum of squares is known.
template <typename T>
__global__ void __launch_bounds__(512) splitk_rms_norm_x4_kernel(T* __restrict__ normed, T* __restrict__ value,
                                                                 const float* __restrict__ partial, int splits,
                                                                 const float* __restrict__ bias, const T* __restrict__ residual,
                                                                 const float* __restrict__ weight, int rows, int width, float eps) {
  // The norm's weight and the bias are the model's: written when it was loaded, like the
  // products' weights, so they are read before the wait for the kernel before (the weight is
  // read once a step and comes from DRAM, which takes longer than the sums from L2).
  dependent_launch_trigger();
  const int quads = width / 4;
  float w_first[4] = {0.f, 0.f, 0.f, 0.f}, b_first[4] = {0.f, 0.f, 0.f, 0.f};
  if ((int)threadIdx.x < quads) {
    load4(weight + 4 * threadIdx.x, w_first);
    if (bias != nullptr) load4(bias + 4 * threadIdx.x, b_first);
  }
  dependent_launch_wait();
  extern __shared__ float row_values[];
  __shared__ float reduce[32];
  const int row = blockIdx.x;
  const size_t plane4 = (size_t)rows * quads;
  const float4* part4 = (const float4*)partial;
  float squares = 0.f;
  float first[4] = {0.f, 0.f, 0.f, 0.f};
  for (int c = threadIdx.x; c < quads; c += blockDim.x) {
    const size_t at4 = (size_t)row * quads + c;
    float res[4] = {0.f, 0.f, 0.f, 0.f};
    if (residual != nullptr) load4(residual + (size_t)row * width + 4 * c, res);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 12 <= splits; s += 12) {
      float4 p[12];
#pragma unroll
      for (int j = 0; j < 12; ++j) p[j] = part4[(size_t)(s + j) * plane4 + at4];
#pragma unroll
      for (int j = 0; j < 12; ++j) {
        v.x += p[j].x; v.y += p[j].y; v.z += p[j].z; v.w += p[j].w;
      }
    }
    for (; s + 4 <= splits; s += 4) {
      float4 p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) p[j] = part4[(size_t)(s + j) * plane4 + at4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v.x += p[j].x; v.y += p[j].y; v.z += p[j].z; v.w += p[j].w;
      }
    }
    for (; s < splits; ++s) {
      const float4 p = part4[(size_t)s * plane4 + at4];
      v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
    }
    float e[4] = {v.x, v.y, v.z, v.w};
    const bool is_first = c == (int)threadIdx.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (bias != nullptr) e[j] += is_first ? b_first[j] : bias[4 * c + j];
      if (residual != nullptr) e[j] += res[j];
      e[j] = to_float(from_float<T>(e[j]));
      squares += e[j] * e[j];
    }
    store4(value + (size_t)row * width + 4 * c, e);
    if (is_first) {
#pragma unroll
      for (int j = 0; j < 4; ++j) first[j] = e[j];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) row_values[4 * c + j] = e[j];
    }
  }
  squares = warp_sum(squares);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) reduce[warp] = squares;
  __syncthreads();
  float total = 0.f;                            // every thread adds the warps' sums in the warps' order
  for (int w = 0; w < warps; ++w) total += reduce[w];
  const float scale = rsqrtf(total / (float)width + eps);
  if ((int)threadIdx.x < quads) {
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = first[j] * scale * w_first[j];
    store4(normed + (size_t)row * width + 4 * threadIdx.x, o);
  }
  for (int i = 4 * blockDim.x + threadIdx.x; i < width; i += blockDim.x)      // rows wider than four columns a thread
    normed[(size_t)row * width + i] = from_float<T>(row_values[i] * scale * weight[i]);
}

// out[t, i] = silu(g) * u with g, u the rounded sums of columns i and inter + i.
template <typename T>
__global__ void splitk_silu_mul_kernel(T* __restrict__ out, const float* __restrict__ partial, int splits, int tokens,
                                       int inter, int block) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * inter) return;
  const long long t = i / inter;
  const int c = (int)(i - t * inter);
  const size_t plane = (size_t)tokens * 2 * inter;
  // block 0: gate in columns [0, I), up in [I, 2I); block b > 0: b gate columns, b up columns, and so on.
  const int gate_col = block > 0 ? (c / block) * 2 * block + c % block : c;
  const int up_col = block > 0 ? gate_col + block : inter + c;
  const float g = to_float(from_float<T>(split_sum(partial, splits, plane, (size_t)t * 2 * inter + gate_col)));
  const float u = to_float(from_float<T>(split_sum(partial, splits, plane, (size_t)t * 2 * inter + up_col)));
  out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// qkv[t, head, :] = round(sum + bias), q and k rotated, k and v written to their pages
// (same arithmetic as rotary_qk_cache_write_kernel of elementwise.cu).
template <typename T>
__global__ void splitk_rotary_cache_write_kernel(T* __restrict__ qkv, const float* __restrict__ partial, int splits,
                                                 const float* __restrict__ bias, const float* __restrict__ table,
                                                 const int* __restrict__ slots, T* __restrict__ keys, T* __restrict__ values,
                                                 int tokens, int heads, int kv_heads, int d, int page_size) {
  dependent_launch_prologue();
  const int half = d >> 1;
  const int all_heads = heads + 2 * kv_heads;
  const int per_token = all_heads * half;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool mine = i < (long long)tokens * per_token;
  const int t = mine ? (int)(i / per_token) : 0;
  const int rest = mine ? (int)(i - (long long)t * per_token) : 0;
  const int head = rest / half, f = rest - head * half;
  const bool to_page = mine && head >= heads && slots != nullptr;
  const int slot = to_page ? slots[t] : -1;
  float bias_lo = 0.f, bias_hi = 0.f;
  if (mine && bias != nullptr) {
    bias_lo = bias[head * d + f];
    bias_hi = bias[head * d + f + half];
  }
  if (!mine) return;
  // Everything is asked for before the sums are waited for: bias, angle, slot.
  const size_t plane = (size_t)tokens * all_heads * d;
  const size_t at = ((size_t)t * all_heads + head) * d;
  const bool rotate = head < heads + kv_heads && table != nullptr;
  const float c = rotate ? table[(size_t)t * d + f] : 1.f, sn = rotate ? table[(size_t)t * d + half + f] : 0.f;
  float lo = split_sum(partial, splits, plane, at + f);
  float hi = split_sum(partial, splits, plane, at + f + half);
  lo = to_float(from_float<T>(lo + bias_lo));
  hi = to_float(from_float<T>(hi + bias_hi));
  if (rotate) {
    rotate_pair(lo, hi, c, sn);
  }
  qkv[at + f] = from_float<T>(lo);
  qkv[at + f + half] = from_float<T>(hi);
  if (slot >= 0 && slot_in_pool(slot, page_size)) {
    const int page = slot / page_size, offset = slot - page * page_size;
    const bool is_key = head < heads + kv_heads;
    const int kv_head = is_key ? head - heads : head - heads - kv_heads;
    T* to = (is_key ? keys : values) + (((size_t)page * kv_heads + kv_head) * page_size + offset) * d;
    to[f] = from_float<T>(lo);
    to[f + half] = from_float<T>(hi);
  }
}

}  // namespace

PAE_EXPORT int pae_splitk_rms_norm(void* normed, void* value, const float* partial, int splits, const float* bias,
                                   const void* residual, const float* weight, int rows, int width, float eps, int dtype,
                                   void* stream) {
  if (rows == 0) return 0;
  if ((size_t)width * sizeof(float) > 160 * 1024) return fail(2, "splitk_rms_norm: rows of %d do not fit shared memory", width);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t bytes = (size_t)width * sizeof(float);
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 384 : (width >= 256 ? 128 : 64));
  const bool by_four = width % 4 == 0 && (((uintptr_t)partial | (uintptr_t)normed | (uintptr_t)value | (uintptr_t)residual |
                                            (uintptr_t)weight | (uintptr_t)bias) & 15) == 0;
  if (dtype == kBF16) {
    auto kernel = by_four ? splitk_rms_norm_x4_kernel<__nv_bfloat16> : splitk_rms_norm_kernel<__nv_bfloat16>;
    if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    launch_kernel(kernel, rows, threads, bytes, s, (__nv_bfloat16*)normed, (__nv_bfloat16*)value, partial, splits, bias,
                                        (const __nv_bfloat16*)residual, weight, rows, width, eps);
  } else if (dtype == kF32) {
    auto kernel = by_four ? splitk_rms_norm_x4_kernel<float> : splitk_rms_norm_kernel<float>;
    if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    launch_kernel(kernel, rows, threads, bytes, s, (float*)normed, (float*)value, partial, splits, bias, (const float*)residual, weight,
                                        rows, width, eps);
  } else {
    return fail(1, "splitk_rms_norm: unknown dtype %d", dtype);
  }
  return check_launch("splitk_rms_norm");
}

PAE_EXPORT int pae_splitk_silu_mul(void* out, const float* partial, int splits, int tokens, int inter, int block,
                                   int dtype, void* stream) {
  const long long n = (long long)tokens * inter;
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kBF16)
    launch_kernel(splitk_silu_mul_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, partial, splits, tokens, inter, block);
  else if (dtype == kF32)
    launch_kernel(splitk_silu_mul_kernel<float>, blocks, 256, 0, s, (float*)out, partial, splits, tokens, inter, block);
  else
    return fail(1, "splitk_silu_mul: unknown dtype %d", dtype);
  return check_launch("splitk_silu_mul");
}

PAE_EXPORT int pae_splitk_rotary_cache_write(void* qkv, const float* partial, int splits, const float* bias,
                                             const float* table, const int* slots, void* keys, void* values, int tokens,
                                             int heads, int kv_heads, int d, int page_size, int dtype, void* stream) {
  if (d % 2) return fail(2, "splitk_rotary_cache_write: head_dim %d is odd", d);
  const long long n = (long long)tokens * (heads + 2 * kv_heads) * (d / 2);
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 127) / 128);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kBF16)
    launch_kernel(splitk_rotary_cache_write_kernel<__nv_bfloat16>, blocks, 128, 0, s, (__nv_bfloat16*)qkv, partial, splits, bias, table, slots, (__nv_bfloat16*)keys, (__nv_bfloat16*)values, tokens, heads, kv_heads, d, page_size);
  else if (dtype == kF32)
    launch_kernel(splitk_rotary_cache_write_kernel<float>, blocks, 128, 0, s, (float*)qkv, partial, splits, bias, table, slots, (float*)keys, (float*)values, tokens, heads, kv_heads, d, page_size);
  else
    return fail(1, "splitk_rotary_cache_write: unknown dtype %d", dtype);
  return check_launch("splitk_rotary_cache_write");
}

PAE_DEFINE_LAST_ERROR()

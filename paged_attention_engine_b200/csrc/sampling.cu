// Sampling on the device from float32 logits: greedy, and temperature by the Gumbel-max
// rule. The reference samples greedily on the host, one argmax and one device-to-host
// read per row (engine/scheduler.py:610); temperature sampling has no counterpart there.
//
// Row r takes token argmax_j (logits[r, j] / T_r + g_j) with g_j = -log(-log(u_j)) and
// u_j a uniform number in (0, 1) that is a pure function of (seed, request key, index of
// the output token, j): a counter-based generator, so the draw does not depend on what
// else is in the batch, on how the prompt was cut, or on a preemption in between.
// T_r == 0 is plain argmax; ties go to the lowest index.
#include "common.cuh"

#include <cfloat>

using namespace pae;

namespace {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x85EBCA6Bu;
  x ^= x >> 13;
  x *= 0xC2B2AE35u;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ bool better(float v, int i, float best, int best_i) {
  return v > best || (v == best && i < best_i);
}

constexpr int THREADS = 512;
constexpr int CHUNK = 4096;      // vocabulary entries per block of the first stage

// Where a sampled token also goes so that the next step's embedding finds it on the device:
// last_token[state_slot[seq_index[logit_rows[r]]]] (engine/scheduler.py:610 reads every token
// back before it goes on; here only the host's copy waits). All null: nowhere.
struct Scatter {
  int* last_token;
  const int* logit_rows;
  const int* seq_index;
  const int* state_slot;
};
__device__ __forceinline__ void keep(int* tokens, const Scatter& to, int r, int token) {
  tokens[r] = token;
  if (to.last_token != nullptr) to.last_token[to.state_slot[to.seq_index[to.logit_rows[r]]]] = token;
}

struct Best {
  float value;
  int index;
};

__device__ __forceinline__ Best block_best(float v_best, int i_best, float* best_v, int* best_i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v_best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i_best, o);
    if (better(ov, oi, v_best, i_best)) {
      v_best = ov;
      i_best = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) {
    best_v[warp] = v_best;
    best_i[warp] = i_best;
  }
  __syncthreads();
  if (warp == 0) {
    v_best = lane < warps ? best_v[lane] : -FLT_MAX;
    i_best = lane < warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v_best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i_best, o);
      if (better(ov, oi, v_best, i_best)) {
        v_best = ov;
        i_best = oi;
      }
    }
  }
  return Best{v_best, i_best};      // valid in lane 0 of warp 0
}

// First stage: the best candidate of one chunk of one row. With a single chunk the token is
// written at once.
__global__ void __launch_bounds__(THREADS) sample_chunks_kernel(int* __restrict__ tokens, float* __restrict__ chunk_value,
                                                                int* __restrict__ chunk_index,
                                                                const float* __restrict__ logits,
                                                                const float* __restrict__ temperature,
                                                                const int* __restrict__ seed_lo, const int* __restrict__ seed_hi,
                                                                const int* __restrict__ request_key,
                                                                const int* __restrict__ output_index, int vocab, int chunks, const Scatter to) {
  dependent_launch_prologue();
  __shared__ float best_v[THREADS / 32];
  __shared__ int best_i[THREADS / 32];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const float t = temperature[r];
  uint32_t h = 0;
  if (t > 0.f) {
    h = mix32((uint32_t)seed_lo[r] ^ 0x9E3779B9u);
    h = mix32(h ^ (uint32_t)seed_hi[r]);
    h = mix32(h + (uint32_t)request_key[r] * 0x7FEB352Du);
    h = mix32(h + (uint32_t)output_index[r] * 0x846CA68Bu);
  }
  const float inv_t = t > 0.f ? 1.f / t : 1.f;
  float v_best = -FLT_MAX;
  int i_best = 0x7fffffff;
  const int end = min(vocab, (chunk + 1) * CHUNK);
  for (int j = chunk * CHUNK + threadIdx.x; j < end; j += THREADS) {
    float v = row[j];
    if (t > 0.f) {
      const uint32_t hv = mix32(h + (uint32_t)j * 0x9E3779B1u);
      const float u = ((float)(hv >> 9) + 0.5f) * (1.0f / 8388608.0f);
      v = v * inv_t - logf(-logf(u));
    }
    if (better(v, j, v_best, i_best)) {
      v_best = v;
      i_best = j;
    }
  }
  const Best best = block_best(v_best, i_best, best_v, best_i);
  if (threadIdx.x == 0) {
    if (chunks == 1) {
      keep(tokens, to, r, best.index == 0x7fffffff ? 0 : best.index);
    } else {
      chunk_value[(size_t)r * chunks + chunk] = best.value;
      chunk_index[(size_t)r * chunks + chunk] = best.index;
    }
  }
}

// Second stage: the best of a row's chunks (ties to the lowest index, as within a chunk).
__global__ void sample_rows_kernel(int* __restrict__ tokens, const float* __restrict__ chunk_value,
                                   const int* __restrict__ chunk_index, int chunks, const Scatter to) {
  dependent_launch_prologue();
  __shared__ float best_v[4];
  __shared__ int best_i[4];
  const int r = blockIdx.x;
  float v_best = -FLT_MAX;
  int i_best = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const float v = chunk_value[(size_t)r * chunks + c];
    const int i = chunk_index[(size_t)r * chunks + c];
    if (better(v, i, v_best, i_best)) {
      v_best = v;
      i_best = i;
    }
  }
  const Best best = block_best(v_best, i_best, best_v, best_i);
  if (threadIdx.x == 0) keep(tokens, to, r, best.index == 0x7fffffff ? 0 : best.index);
}

}  // namespace

// Words (4 bytes each) of scratch that pae_sample needs.
PAE_EXPORT long long pae_sample_scratch_words(int rows, int vocab) {
  const int chunks = (vocab + CHUNK - 1) / CHUNK;
  return chunks > 1 ? 2LL * rows * chunks : 0;
}

// tokens int32 [rows]; logits float32 [rows, vocab]; per row: temperature (float32),
// the two halves of the 64-bit seed, the request's key and the index of the output token.
// `scratch` holds pae_sample_scratch_words(rows, vocab) words (may be null when that is 0).
// With `last_token` (and the step's logit_rows, seq_index, state_slot) the token of row r is also
// written to last_token[state_slot[seq_index[logit_rows[r]]]]; null leaves that to the caller.
PAE_EXPORT int pae_sample(int* tokens, const float* logits, const float* temperature, const int* seed_lo,
                          const int* seed_hi, const int* request_key, const int* output_index, int rows, int vocab,
                          void* scratch, int* last_token, const int* logit_rows, const int* seq_index,
                          const int* state_slot, void* stream) {
  if (rows == 0) return 0;
  if (vocab < 1) return fail(2, "sample: vocabulary of %d", vocab);
  if (rows > 65535) return fail(3, "sample: %d rows are more than one launch takes", rows);
  const int chunks = (vocab + CHUNK - 1) / CHUNK;
  if (chunks > 1 && scratch == nullptr) return fail(2, "sample: no scratch for %d chunks", chunks);
  if (last_token != nullptr && (logit_rows == nullptr || seq_index == nullptr || state_slot == nullptr))
    return fail(2, "sample: tokens are to be kept for the next step, but the step's rows, entries or slots are missing");
  const Scatter to{last_token, logit_rows, seq_index, state_slot};
  float* chunk_value = (float*)scratch;
  int* chunk_index = (int*)scratch + (size_t)rows * chunks;
  cudaStream_t s = (cudaStream_t)stream;
  launch_kernel(sample_chunks_kernel, dim3(chunks, rows), THREADS, 0, s, tokens, chunk_value, chunk_index, logits, temperature, seed_lo,
                                                             seed_hi, request_key, output_index, vocab, chunks, to);
  if (int err = check_launch("sample")) return err;
  if (chunks > 1) {
    launch_kernel(sample_rows_kernel, rows, 128, 0, s, tokens, chunk_value, chunk_index, chunks, to);
    return check_launch("sample");
  }
  return 0;
}

PAE_DEFINE_LAST_ERROR()

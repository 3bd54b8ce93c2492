// Attention over the paged cache for the bfloat16 path (kernels and launch helpers;
// the exported entry points are in attention_mma.cu), on tensor cores (mma.sync
// m16n8k16 with float32 accumulation), reading keys and values in place through the block
// table. Two kernels and a merge:
//
//   decode   requests that bring ONE token. One warp owns one (request, kv head, slice of
//            the keys): the query heads that share the kv head are the 16 rows of the MMA
//            (grouped-query attention without repeating keys: the reference copies them,
//            engine/attention.py:46-74), so every key and value is read from memory once
//            per kv head. The keys of a request are cut into slices so that a small batch
//            still fills the machine; each slice leaves an unnormalised output with its
//            running maximum and sum in float32 scratch, and `merge` combines the slices
//            of a (request, head) in their order.
//   prefill  requests that bring several tokens (a portion of a prompt at any offset). A
//            block owns 64 consecutive query tokens of one request and one head, four
//            warps of 16 rows each, and walks that request's pages 64 keys at a time with
//            a running softmax.
//
// The rule of engine/attention.py:581-586 is evaluated per score: the query at position p
// sees key j when j <= p and j < kv_len, and p - j < window when the layer has one.
// Scores are scaled in float32; probabilities are rounded to bfloat16 for the second
// product, as the value operand is.
//
// Sizes: head_dim 32, 64 or 128; page sizes that are multiples of 16; up to 16 query
// heads per kv head. Everything else is refused here and runs on the CUDA-core kernel.
#pragma once

#include "common.cuh"


#include <cfloat>
#include <mutex>
#include <set>
#include <utility>

namespace pae_attention {

using namespace pae;


constexpr int TILE_KEYS = 16;            // keys per MMA step of the decode kernel: never straddles a page
// The sliced decode kernel: warps (slices) per block, and tiles of 16 keys that a warp keeps in
// flight. A tile takes about a microsecond to arrive and a slice is a handful of tiles, so a
// slice's time is its number of tiles divided by the depth, in microseconds. Measured at the
// 1.5B shape, context 4096 (decode step, ms at batch 1 / 8 / 64): two stages and four warps
// 1.44 / 1.53 / 2.99; four stages and two warps 1.21 / 1.33 / 2.95; three stages 1.22 / 1.32 /
// 2.89 (four blocks an SM); six stages 1.19 / 1.35 / 3.19.
constexpr int SLICE_WARPS = 2;
constexpr int SLICE_STAGES = 3;
constexpr int PREFILL_BQ = 64;           // query tokens per block
constexpr int PREFILL_BKEYS = 64;        // keys per iteration
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}

__device__ __forceinline__ void mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the special-function unit (two units in the last place; flushes denormals).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// A tile of rows x D bfloat16 in shared memory; the 16-byte chunk c of row r lives at chunk
// c ^ swizzle(r), so that the eight rows an ldmatrix reads fall into different banks.
template <int D>
struct TileLayout {
  static constexpr int CHUNKS = D / 8;                        // 16-byte chunks per row
  static constexpr int SHIFT = CHUNKS >= 8 ? 0 : (CHUNKS == 4 ? 1 : 2);
  static constexpr int MASK = CHUNKS >= 8 ? 7 : CHUNKS - 1;
  __device__ static __forceinline__ int offset_bytes(int row, int chunk) {
    return (row * CHUNKS + (chunk ^ ((row >> SHIFT) & MASK))) * 16;
  }
};

// The A fragments (16 rows x D) of a warp's queries, straight from global memory. Row r of
// the fragment is `row_ptr(r)`, or nothing (zeros) when that returns null.
template <int D, typename RowPtr>
__device__ __forceinline__ void load_query_fragments(uint32_t (*q)[4], RowPtr row_ptr) {
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* r0 = row_ptr(lane >> 2);
  const __nv_bfloat16* r1 = row_ptr((lane >> 2) + 8);
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    q[k][0] = r0 ? *(const uint32_t*)(r0 + k * 16 + c) : 0u;
    q[k][1] = r1 ? *(const uint32_t*)(r1 + k * 16 + c) : 0u;
    q[k][2] = r0 ? *(const uint32_t*)(r0 + k * 16 + 8 + c) : 0u;
    q[k][3] = r1 ? *(const uint32_t*)(r1 + k * 16 + 8 + c) : 0u;
  }
}

// scores[16 x 16] = Q . K^T for 16 keys that start at row `key0` of the K tile.
template <int D>
__device__ __forceinline__ void scores_16_keys(float (*s)[4], const uint32_t (*q)[4], uint32_t k_tile, int key0) {
  const int lane = threadIdx.x & 31;
  const int mid = lane >> 3, r = lane & 7;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    uint32_t b[4];
    // matrices: (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
    ldmatrix_x4(b, k_tile + TileLayout<D>::offset_bytes(key0 + (mid >> 1) * 8 + r, k * 2 + (mid & 1)));
    mma_16816(s[0], q[k], b[0], b[1]);
    mma_16816(s[1], q[k], b[2], b[3]);
  }
}

// out[16 x D] += P[16 x 16] . V for 16 keys that start at row `key0` of the V tile.
template <int D>
__device__ __forceinline__ void accumulate_16_keys(float (*o)[4], const uint32_t* p, uint32_t v_tile, int key0) {
  const int lane = threadIdx.x & 31;
  const int mid = lane >> 3, r = lane & 7;
#pragma unroll
  for (int n = 0; n < D / 16; ++n) {
    uint32_t b[4];
    // matrices (transposed on load): (keys 0-7, dims 0-7), (keys 8-15, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 8-15)
    ldmatrix_x4_trans(b, v_tile + TileLayout<D>::offset_bytes(key0 + (mid & 1) * 8 + r, n * 2 + (mid >> 1)));
    mma_16816(o[2 * n], p, b[0], b[1]);
    mma_16816(o[2 * n + 1], p, b[2], b[3]);
  }
}

// One step of the running softmax for a 16 x 16 block of scores held as two n8 tiles.
// `visible(row_half, key_in_block)` says which scores count. Rows are lane/4 (half 0) and
// lane/4 + 8 (half 1). Returns the probabilities as the A fragment of the next product.
template <int D, typename Visible>
__device__ __forceinline__ void softmax_step(float (*s)[4], float* row_max, float* row_sum, float (*o)[4], uint32_t* p,
                                             float scale_log2, bool unmasked, Visible visible) {
  const int lane = threadIdx.x & 31;
  const int c = (lane & 3) * 2;
  float block_max[2] = {-FLT_MAX, -FLT_MAX};
  if (unmasked) {             // the same for the whole warp: every score of the block counts
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[t][j] *= scale_log2;
        block_max[j >> 1] = fmaxf(block_max[j >> 1], s[t][j]);
      }
  } else {
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int half = j >> 1, key = t * 8 + c + (j & 1);
        s[t][j] = visible(half, key) ? s[t][j] * scale_log2 : -FLT_MAX;
        block_max[half] = fmaxf(block_max[half], s[t][j]);
      }
  }
  float rescale[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    block_max[half] = fmaxf(block_max[half], __shfl_xor_sync(0xffffffffu, block_max[half], 1));
    block_max[half] = fmaxf(block_max[half], __shfl_xor_sync(0xffffffffu, block_max[half], 2));
    const float new_max = fmaxf(row_max[half], block_max[half]);
    rescale[half] = row_max[half] == -FLT_MAX ? 0.f : fast_exp2(row_max[half] - new_max);
    row_max[half] = new_max;
  }
  float block_sum[2] = {0.f, 0.f};
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int half = j >> 1;
      const float e = s[t][j] == -FLT_MAX ? 0.f : fast_exp2(s[t][j] - row_max[half]);
      s[t][j] = e;
      block_sum[half] += e;
    }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    block_sum[half] += __shfl_xor_sync(0xffffffffu, block_sum[half], 1);
    block_sum[half] += __shfl_xor_sync(0xffffffffu, block_sum[half], 2);
    row_sum[half] = row_sum[half] * rescale[half] + block_sum[half];
  }
  // The running output only has to be rescaled when some row's maximum moved (multiplying
  // by exactly 1 changes nothing); late in a long row that is rare.
  if (__any_sync(0xffffffffu, rescale[0] != 1.f || rescale[1] != 1.f)) {
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o[n][0] *= rescale[0];
      o[n][1] *= rescale[0];
      o[n][2] *= rescale[1];
      o[n][3] *= rescale[1];
    }
  }
  p[0] = pack_bf16(s[0][0], s[0][1]);
  p[1] = pack_bf16(s[0][2], s[0][3]);
  p[2] = pack_bf16(s[1][0], s[1][1]);
  p[3] = pack_bf16(s[1][2], s[1][3]);
}

// ---------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* qkv;     // [tokens, heads + 2 kv_heads, D]
  const __nv_bfloat16* keys;    // [pages, kv_heads, page_size, D]
  const __nv_bfloat16* values;
  const int* block_table;
  const int* q_start;
  const int* kv_len;
  float* part_out;              // [tokens?]: [request, head, slice, D]
  float* part_max;              // [request, head, slice]  (in units of log2)
  float* part_sum;
  int table_width, heads, kv_heads, page_size, window;
  int slice_keys;               // keys per slice, a multiple of 16
  int max_slices;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(SLICE_WARPS * 32) decode_slices_kernel(const DecodeParams p) {
  // The step's integers (starts, lengths, block tables) were copied in before the step began
  // and the keys and values of EARLIER tokens are not written by any kernel of this step, so
  // a slice's first tiles are fetched before the wait for the kernel that precedes this one
  // (which writes this step's queries, keys and values). Every block waits before it leaves.
  dependent_launch_trigger();
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slice = blockIdx.x * SLICE_WARPS + warp;
  const int g = blockIdx.y, b = blockIdx.z;
  const int token = p.q_start[b];
  const int kv_len = p.kv_len[b];
  const int first_key = p.window > 0 ? max(0, kv_len - p.window) : 0;     // the query stands at kv_len - 1
  const int base = (first_key / TILE_KEYS) * TILE_KEYS;
  const int begin = base + slice * p.slice_keys;
  const int end = min(kv_len, begin + p.slice_keys);
  if (p.q_start[b + 1] - token != 1 || slice >= p.max_slices || begin >= kv_len) {   // nothing for this warp
    dependent_launch_wait();
    return;
  }

  const int groups = p.heads / p.kv_heads;
  const int row_elems = (p.heads + 2 * p.kv_heads) * D;
  constexpr int TILE_BYTES = TILE_KEYS * D * 2;
  uint8_t* mine = smem + warp * SLICE_STAGES * 2 * TILE_BYTES;      // stages of (K tile, V tile)
  const uint32_t mine_u32 = smem_u32(mine);
  const int* table = p.block_table + (size_t)b * p.table_width;

  auto fetch = [&](int stage, int key0) {
    const int page = checked_page(table[checked_table_index(key0 / p.page_size, p.table_width)]);
    const size_t row0 = ((size_t)page * p.kv_heads + g) * p.page_size + (key0 % p.page_size);
    const uint32_t k_dst = mine_u32 + stage * 2 * TILE_BYTES;
    constexpr int CHUNKS = TILE_KEYS * D / 8;
#pragma unroll
    for (int i = lane; i < CHUNKS; i += 32) {
      const int row = i / (D / 8), c = i % (D / 8);
      const int off = TileLayout<D>::offset_bytes(row, c);
      cp_async16(k_dst + off, p.keys + (row0 + row) * D + c * 8);
      cp_async16(k_dst + TILE_BYTES + off, p.values + (row0 + row) * D + c * 8);
    }
  };

  // Tiles 0 .. SLICE_STAGES - 2 start the pipeline, one commit group each; those that hold
  // earlier tokens only are asked for before the wait.
  const int tiles = (end - begin + TILE_KEYS - 1) / TILE_KEYS;
  int early = 0;
  while (early < SLICE_STAGES - 1 && early < tiles && begin + (early + 1) * TILE_KEYS <= kv_len - 1) {
    fetch(early, begin + early * TILE_KEYS);
    cp_async_commit();
    ++early;
  }
  dependent_launch_wait();
  uint32_t q[D / 16][4];
  load_query_fragments<D>(q, [&](int r) -> const __nv_bfloat16* {
    return r < groups ? p.qkv + (size_t)token * row_elems + (size_t)(g * groups + r) * D : nullptr;
  });
  for (int i = early; i < SLICE_STAGES - 1; ++i) {
    if (i < tiles) fetch(i, begin + i * TILE_KEYS);
    cp_async_commit();
  }

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float row_max[2] = {-FLT_MAX, -FLT_MAX}, row_sum[2] = {0.f, 0.f};

  for (int t = 0; t < tiles; ++t) {
    // The stage that tile t + SLICE_STAGES - 1 goes to held tile t - 1, which is read (the
    // __syncwarp that ends every round). One commit group per round, empty or not, so that
    // "all but the newest SLICE_STAGES - 1 groups" always means "tile t has arrived".
    const int ahead = t + SLICE_STAGES - 1;
    if (ahead < tiles) fetch(ahead % SLICE_STAGES, begin + ahead * TILE_KEYS);
    cp_async_commit();
    cp_async_wait<SLICE_STAGES - 1>();
    __syncwarp();
    const uint32_t k_tile = mine_u32 + (t % SLICE_STAGES) * 2 * TILE_BYTES;
    const int key0 = begin + t * TILE_KEYS;
    float s[2][4];
    scores_16_keys<D>(s, q, k_tile, 0);
    uint32_t pa[4];
    softmax_step<D>(s, row_max, row_sum, o, pa, p.scale_log2, key0 >= first_key && key0 + TILE_KEYS <= end,
                    [&](int, int key) { return key0 + key >= first_key && key0 + key < end; });
    accumulate_16_keys<D>(o, pa, k_tile + TILE_BYTES, 0);
    __syncwarp();      // the tile is read; the next iteration's fetch may overwrite the other stage
  }
  cp_async_wait<0>();

  // Rows 0..groups-1 are real heads. Row lane/4 (half 0) and lane/4 + 8 (half 1).
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = (lane >> 2) + half * 8;
    if (r >= groups) continue;
    const size_t at = ((size_t)b * p.heads + g * groups + r) * p.max_slices + slice;
    float* out = p.part_out + at * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *(float2*)(out + n * 8 + (lane & 3) * 2) = make_float2(o[n][half * 2], o[n][half * 2 + 1]);
    if ((lane & 3) == 0) {
      p.part_max[at] = row_max[half];
      p.part_sum[at] = row_sum[half];
    }
  }
}

// out[token, head, :] = sum_s w_s part_out[s] / sum_s w_s part_sum[s], w_s = 2^(max_s - max).
// One block of four warps per (request, head). Everything the block needs is asked for before
// anything is waited for: a thread's slice maxima and sums, and the partial outputs of the
// slices its warp folds (warp w takes slices w, w + 4, ...; a lane owns D / 32 neighbouring
// dimensions), twenty-four slices per warp at a time (96 in all: the most that a step of few
// requests is cut into; with sixteen, the 74 slices of batch 8 at context 4,096 cost a warp a
// further trip to memory). The weights are then worked out once into
// shared memory, each warp folds its slices in their order, and the warps' sums are added in
// the order of the warps, so the result does not depend on timing.
constexpr int MERGE_WARPS = 4;
constexpr int MERGE_DEPTH = 24;      // slices per warp whose partial outputs are in registers at one time

template <int D>
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_slices_kernel(
    __nv_bfloat16* __restrict__ out, const float* __restrict__ part_out, const float* __restrict__ part_max,
    const float* __restrict__ part_sum, const int* __restrict__ q_start, const int* __restrict__ kv_len, int heads, int window,
    int slice_keys, int max_slices) {
  // The kernel before this one is the sliced decode kernel of the same call, which has read
  // the step's integers itself: they are read before the wait.
  dependent_launch_trigger();
  extern __shared__ float weights[];          // [max_slices], then [MERGE_WARPS][D]
  __shared__ float reduce[2 * MERGE_WARPS];
  const int h = blockIdx.x, b = blockIdx.y;
  const int token = q_start[b];
  const bool single = q_start[b + 1] - token == 1;
  const int n_kv = kv_len[b];
  dependent_launch_wait();
  if (!single) return;
  const int first_key = window > 0 ? max(0, n_kv - window) : 0;
  const int base = (first_key / TILE_KEYS) * TILE_KEYS;
  const int slices = min(max_slices, (n_kv - base + slice_keys - 1) / slice_keys);
  const size_t at = ((size_t)b * heads + h) * max_slices;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int PER_LANE = D / 32;

  // ---- requests: this warp's first MERGE_DEPTH partial outputs, then the maxima and sums
  float part[MERGE_DEPTH][PER_LANE];
#pragma unroll
  for (int i = 0; i < MERGE_DEPTH; ++i) {
    const int s = warp + i * MERGE_WARPS;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) part[i][j] = 0.f;
    if (s < slices) {
      const float* from = part_out + (at + s) * D + lane * PER_LANE;
      if (PER_LANE == 4) {
        const float4 v = *(const float4*)from;
        part[i][0] = v.x; part[i][1] = v.y; part[i][2] = v.z; part[i][3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) part[i][j] = from[j];
      }
    }
  }
  float top = -FLT_MAX;
  for (int s = threadIdx.x; s < slices; s += blockDim.x) {
    const float m = part_max[at + s];
    weights[s] = m;
    top = fmaxf(top, m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
  if (lane == 0) reduce[warp] = top;
  __syncthreads();
  top = reduce[0];
#pragma unroll
  for (int w = 1; w < MERGE_WARPS; ++w) top = fmaxf(top, reduce[w]);

  float total = 0.f;
  for (int s = threadIdx.x; s < slices; s += blockDim.x) {
    const float w = exp2f(weights[s] - top);    // this thread wrote weights[s] itself
    weights[s] = w;
    total += part_sum[at + s] * w;
  }
  total = warp_sum(total);
  if (lane == 0) reduce[MERGE_WARPS + warp] = total;
  __syncthreads();                              // the weights of all slices and the warps' sums are in place
  total = 0.f;
#pragma unroll
  for (int w = 0; w < MERGE_WARPS; ++w) total += reduce[MERGE_WARPS + w];
  const float inv = total > 0.f ? 1.f / total : 0.f;

  // ---- this warp's slices in their order
  float acc[PER_LANE];
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) acc[j] = 0.f;
#pragma unroll
  for (int i = 0; i < MERGE_DEPTH; ++i) {
    const int s = warp + i * MERGE_WARPS;
    if (s < slices) {
      const float w = weights[s];
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j) acc[j] += part[i][j] * w;
    }
  }
  for (int s = warp + MERGE_DEPTH * MERGE_WARPS; s < slices; s += MERGE_WARPS) {     // more than 96 slices
    const float w = weights[s];
    const float* from = part_out + (at + s) * D + lane * PER_LANE;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) acc[j] += from[j] * w;
  }
  float* across = weights + max_slices;          // [MERGE_WARPS][D]
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) across[warp * D + lane * PER_LANE + j] = acc[j];
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < MERGE_WARPS; ++w) v += across[w * D + d];
    out[((size_t)token * heads + h) * D + d] = __float2bfloat16_rn(v * inv);
  }
}

// ---------------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------------
struct PrefillParams {
  __nv_bfloat16* out;           // [tokens, heads, D]
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* keys;
  const __nv_bfloat16* values;
  const int* block_table;
  const int* q_start;
  const int* q_pos0;
  const int* kv_len;
  int table_width, heads, kv_heads, page_size, window;
  int skip_single;              // requests of one token are left to the decode kernel
  const int* work_index;        // the requests that this launch works on, one per grid z (null: request z)
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(128) prefill_kernel(const PrefillParams p) {
  dependent_launch_prologue();
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = p.work_index != nullptr ? p.work_index[blockIdx.z] : (int)blockIdx.z;
  const int first_token = p.q_start[b];
  const int q_count = p.q_start[b + 1] - first_token;
  if (p.skip_single && q_count == 1) return;
  // A block takes two 64-token tiles of its request, the x-th from the end and the x-th from
  // the start: a late tile sees many keys and an early one few, so every block of a request
  // has about the same work.
  const int q_tiles = (q_count + PREFILL_BQ - 1) / PREFILL_BQ;
  if ((int)blockIdx.x * 2 >= q_tiles) return;
  const uint32_t smem_base = smem_u32(smem);
  const int g = h / (p.heads / p.kv_heads);
  const int row_elems = (p.heads + 2 * p.kv_heads) * D;
  const int* table = p.block_table + (size_t)b * p.table_width;
  const int warp_row0 = warp * 16;
  constexpr int TILE_BYTES = PREFILL_BKEYS * D * 2;
  constexpr int ROW_CHUNKS = D / 8;
  constexpr int ROWS_PER_PASS = 128 / ROW_CHUNKS;
  constexpr int PER_THREAD = PREFILL_BKEYS / ROWS_PER_PASS;
  const int my_chunk = threadIdx.x % ROW_CHUNKS, my_row = threadIdx.x / ROW_CHUNKS;
  int dst_offset[PER_THREAD];
#pragma unroll
  for (int j = 0; j < PER_THREAD; ++j) dst_offset[j] = TileLayout<D>::offset_bytes(my_row + j * ROWS_PER_PASS, my_chunk);
  const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? __ffs(p.page_size) - 1 : -1;
  const size_t head_offset = (size_t)g * p.page_size * D + my_chunk * 8;
  const size_t page_stride = (size_t)p.kv_heads * p.page_size * D;

#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
  const int tile = pass == 0 ? q_tiles - 1 - (int)blockIdx.x : (int)blockIdx.x;
  if (pass == 1 && tile == q_tiles - 1 - (int)blockIdx.x) break;      // the middle tile of an odd count
  const int rows = min(PREFILL_BQ, q_count - tile * PREFILL_BQ);
  const int pos0 = p.q_pos0[b] + tile * PREFILL_BQ;             // position of the block's first query
  const int kv_end = min(p.kv_len[b], pos0 + rows);
  const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kv_begin = (first_key / TILE_KEYS) * TILE_KEYS;
  uint32_t q[D / 16][4];
  load_query_fragments<D>(q, [&](int r) -> const __nv_bfloat16* {
    const int row = warp_row0 + r;
    return row < rows ? p.qkv + (size_t)(first_token + tile * PREFILL_BQ + row) * row_elems + (size_t)h * D : nullptr;
  });

  // All 128 threads bring a tile of 64 keys and values; keys past kv_end are zero-filled rows
  // that the mask never lets through (their pages may not exist). A thread copies the same
  // 16-byte column of PER_THREAD rows in every tile, so where they go in shared memory is
  // worked out once.
  auto fetch = [&](int stage, int key0) {
    const uint32_t k_dst = smem_base + stage * 2 * TILE_BYTES;
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
      const int key = key0 + my_row + j * ROWS_PER_PASS;
      if (key < kv_end) {
        int page, offset;
        if (page_shift >= 0) {
          page = table[checked_table_index(key >> page_shift, p.table_width)];
          offset = key & (p.page_size - 1);
        } else {
          page = table[checked_table_index(key / p.page_size, p.table_width)];
          offset = key % p.page_size;
        }
        page = checked_page(page);
        const size_t src = (size_t)page * page_stride + head_offset + (size_t)offset * D;
        cp_async16(k_dst + dst_offset[j], p.keys + src);
        cp_async16(k_dst + TILE_BYTES + dst_offset[j], p.values + src);
      } else {
        *(uint4*)(smem + stage * 2 * TILE_BYTES + dst_offset[j]) = make_uint4(0, 0, 0, 0);
        *(uint4*)(smem + stage * 2 * TILE_BYTES + TILE_BYTES + dst_offset[j]) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float row_max[2] = {-FLT_MAX, -FLT_MAX}, row_sum[2] = {0.f, 0.f};
  const int my_pos[2] = {pos0 + warp_row0 + (lane >> 2), pos0 + warp_row0 + (lane >> 2) + 8};
  const int warp_last_pos = warp_row0 < rows ? pos0 + min(rows, warp_row0 + 16) - 1 : -1;   // -1: the warp has no rows

  const int tiles = (kv_end - kv_begin + PREFILL_BKEYS - 1) / PREFILL_BKEYS;
  fetch(0, kv_begin);
  cp_async_commit();
  for (int t = 0; t < tiles; ++t) {
    if (t + 1 < tiles) fetch((t + 1) & 1, kv_begin + (t + 1) * PREFILL_BKEYS);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t k_tile = smem_base + (t & 1) * 2 * TILE_BYTES;
    const int tile_key0 = kv_begin + t * PREFILL_BKEYS;
#pragma unroll
    for (int sub = 0; sub < PREFILL_BKEYS / 16; ++sub) {
      const int key0 = tile_key0 + sub * 16;
      // Nothing of these 16 keys is visible to this warp's rows: too late, too early, or no rows.
      if (key0 > warp_last_pos || key0 >= kv_end) continue;
      if (p.window > 0 && key0 + 15 < pos0 + warp_row0 - p.window + 1) continue;
      float s[2][4];
      scores_16_keys<D>(s, q, k_tile, sub * 16);
      uint32_t pa[4];
      // Keys wholly before the warp's first row, inside every row's window and inside the
      // request need no mask.
      const bool unmasked = key0 + 15 <= pos0 + warp_row0 && key0 + 16 <= kv_end &&
                            (p.window <= 0 || warp_last_pos - key0 < p.window);
      softmax_step<D>(s, row_max, row_sum, o, pa, p.scale_log2, unmasked, [&](int half, int key) {
        const int j = key0 + key;
        return j < kv_end && j <= my_pos[half] && (p.window <= 0 || my_pos[half] - j < p.window);
      });
      accumulate_16_keys<D>(o, pa, k_tile + TILE_BYTES, sub * 16);
    }
    __syncthreads();     // every warp has read this stage before the next fetch refills it
  }
  cp_async_wait<0>();

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = warp_row0 + (lane >> 2) + half * 8;
    if (row >= rows) continue;
    const float inv = row_sum[half] > 0.f ? 1.f / row_sum[half] : 0.f;
    __nv_bfloat16* out = p.out + ((size_t)(first_token + tile * PREFILL_BQ + row) * p.heads + h) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *(uint32_t*)(out + n * 8 + (lane & 3) * 2) = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
  }
  }  // the block's two tiles
}

// Raises a kernel's dynamic shared memory limit, once per kernel and device (the attribute
// belongs to the kernel as loaded on one device).
template <typename Kernel>
int allow_smem(Kernel kernel, size_t bytes, const char* what) {
  static std::mutex mutex;
  static std::set<std::pair<int, const void*>> done;
  if (bytes <= 48 * 1024) return 0;
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(100, "%s: cudaGetDevice: %s", what, cudaGetErrorString(err));
  std::lock_guard<std::mutex> guard(mutex);
  const std::pair<int, const void*> key(device, (const void*)kernel);
  if (done.count(key)) return 0;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) return fail(100, "%s: %s", what, cudaGetErrorString(err));
  done.insert(key);
  return 0;
}

inline size_t slices_smem_bytes(int d) { return (size_t)SLICE_WARPS * SLICE_STAGES * 2 * TILE_KEYS * d * 2; }

template <int D>
int launch_decode(const DecodeParams& p, __nv_bfloat16* out, int seqs, cudaStream_t s) {
  const size_t bytes = slices_smem_bytes(D);
  if (int err = allow_smem(decode_slices_kernel<D>, bytes, "paged_attention_decode")) return err;
  dim3 grid((p.max_slices + SLICE_WARPS - 1) / SLICE_WARPS, p.kv_heads, seqs);
  launch_kernel(decode_slices_kernel<D>, grid, SLICE_WARPS * 32, bytes, s, p);
  if (int err = check_launch("paged_attention_decode")) return err;
  launch_kernel(merge_slices_kernel<D>, dim3(p.heads, seqs), MERGE_WARPS * 32, (p.max_slices + MERGE_WARPS * D) * sizeof(float), s, out, p.part_out, p.part_max, p.part_sum, p.q_start,
                                                                     p.kv_len, p.heads, p.window, p.slice_keys, p.max_slices);
  return check_launch("paged_attention_merge");
}

template <int D>
int launch_prefill(const PrefillParams& p, int seqs, int max_q_len, cudaStream_t s) {
  const size_t bytes = (size_t)2 * 2 * PREFILL_BKEYS * D * 2;
  if (int err = allow_smem(prefill_kernel<D>, bytes, "paged_attention_prefill")) return err;
  const int q_tiles = (max_q_len + PREFILL_BQ - 1) / PREFILL_BQ;
  dim3 grid((q_tiles + 1) / 2, p.heads, seqs);
  launch_kernel(prefill_kernel<D>, grid, 128, bytes, s, p);
  return check_launch("paged_attention_prefill");
}

inline int check_sizes(const char* what, int heads, int kv_heads, int d, int page_size, int seqs) {
  if (d != 32 && d != 64 && d != 128) return fail(2, "%s: head_dim %d is not 32, 64 or 128", what, d);
  if (page_size < 16 || page_size % 16) return fail(2, "%s: page size %d is not a multiple of 16", what, page_size);
  if (kv_heads < 1 || heads % kv_heads) return fail(2, "%s: %d heads over %d kv heads", what, heads, kv_heads);
  if (heads > 65535 || seqs > 65535) return fail(3, "%s: %d heads x %d requests exceed one launch", what, heads, seqs);
  return 0;
}


// The decode kernel and its merge over caller-given scratch (see pae_paged_attention_decode).
inline int decode_with_scratch(void* out, const void* qkv, const void* keys, const void* values, const int* block_table,
                               int table_width, const int* q_start, const int* kv_len, int seqs, int heads, int kv_heads,
                               int d, int page_size, float scale, int window, int slice_keys, int max_slices,
                               float* scratch, cudaStream_t s) {
  if (seqs == 0) return 0;
  if (int err = check_sizes("paged_attention_decode", heads, kv_heads, d, page_size, seqs)) return err;
  if (heads / kv_heads > 16) return fail(2, "paged_attention_decode: %d query heads per kv head are more than 16", heads / kv_heads);
  if (slice_keys < 16 || slice_keys % 16 || max_slices < 1) return fail(2, "paged_attention_decode: slices of %d keys x %d", slice_keys, max_slices);
  if (scratch == nullptr) return fail(2, "paged_attention_decode: no scratch for the slices' partial results was given");
  // The merge keeps a weight per slice (and a row per warp) in shared memory: refused here, before anything is launched.
  if ((size_t)(max_slices + MERGE_WARPS * d) * sizeof(float) > 40 * 1024)
    return fail(2, "paged_attention_decode: %d slices are more than the merge takes (%d at head size %d)", max_slices,
                (int)(40 * 1024 / sizeof(float)) - MERGE_WARPS * d, d);
  DecodeParams p{};
  p.qkv = (const __nv_bfloat16*)qkv;
  p.keys = (const __nv_bfloat16*)keys;
  p.values = (const __nv_bfloat16*)values;
  p.block_table = block_table;
  p.q_start = q_start;
  p.kv_len = kv_len;
  const size_t rows = (size_t)seqs * heads * max_slices;
  p.part_out = scratch;
  p.part_max = scratch + rows * d;
  p.part_sum = p.part_max + rows;
  p.table_width = table_width;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.page_size = page_size;
  p.window = window;
  p.slice_keys = slice_keys;
  p.max_slices = max_slices;
  p.scale_log2 = scale * LOG2E;
  if (d == 32) return launch_decode<32>(p, (__nv_bfloat16*)out, seqs, s);
  if (d == 64) return launch_decode<64>(p, (__nv_bfloat16*)out, seqs, s);
  return launch_decode<128>(p, (__nv_bfloat16*)out, seqs, s);
}

// Floats of scratch that the decode kernel needs for `seqs` requests and `max_slices` slices.
inline long long decode_scratch_floats(int seqs, int heads, int d, int max_slices) {
  return (long long)seqs * heads * max_slices * (d + 2);
}

}  // namespace pae_attention

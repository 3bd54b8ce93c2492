// The products of a step of few tokens (decoding), each as ONE kernel that leaves finished
// output: no K is split over blocks, so nothing has to be summed by a kernel of its own, and
// what used to follow a product in such a kernel runs in the product's epilogue.
//
// A decode step of a small model is a chain of short kernels, and a link of the chain costs two
// microseconds and more whatever it moves. The tcgen05 products of such a step fill the machine
// by splitting K over blocks, which leaves partial sums and a kernel between every two products
// to add them up (with the norm, the rotation or SiLU x up folded in): ten links a layer. With
// few tokens the tensor cores' width is of no use; what counts is that every SM streams its
// share of the weights. So here a WARP owns 16 weight rows (the 16 rows of an mma.sync
// m16n8k16, the tokens are the columns) and the full K (or a block's warps share K out and add
// up through shared memory, in their order). Which 16 rows makes the epilogue local:
//
//   q|k|v     8 rows of a head's first half and their 8 partners of the second half: the
//             rotation's pairs (j, j + d/2) meet in one thread. Epilogue: RMSNorm's scale of
//             the token (the product runs over x * norm weight; rsqrt(mean x^2 + eps) is one
//             factor per token and is applied to the sums), bias, rounding, rotation, page write.
//   gate|up   8 gate rows and their 8 up rows (the weight's rows alternate in blocks of 16):
//             epilogue = scale, rounding, SiLU(gate) * up.
//   o, down   16 neighbouring rows; epilogue = + residual, rounding.
//
// Weights: every warp runs a ring of its own, filled by TMA and watched through one mbarrier
// per stage. A stage is two to four neighbouring chunks of 64 of K: two copies of 8 rows x 64 x
// chunks each (the lower and the upper eight MMA rows), 128-byte swizzle, which is the layout
// ldmatrix wants. The warp that reads a stage is the warp that asks for the next one into it, so
// the main loop has no block-wide barrier. The first stages are asked for BEFORE the wait for
// the kernel before this one (weights were written when the model was loaded), so they stream
// while that kernel finishes. Plain 16-byte cp.async copies of the same chunks kept too little
// on the way per SM: 1.4 to 2.4 TB/s where the TMA ring streams.
//
// Activations. Where the input is a norm's (q|k|v, gate|up), the block first builds, once, the
// whole operand in shared memory: x * norm weight in float32, rounded to bfloat16, already in the
// order of the MMA's B fragments (one 8-byte load per lane and k-step), and the tokens'
// rsqrt(mean x^2 + eps). Where it is not (o, down), the warps' K ranges differ and the
// activations' chunks [tokens x 64] come through the ring beside the weights' chunks. What the
// epilogue adds (bias, angles and slots, the residual) is asked for before the main loop.
//
// Sizes: K a multiple of 64, at most 24 tokens, head_dim a multiple of 16, and shared memory
// for the ring and a normed operand. Everything else is refused here and runs on the tcgen05
// products and their summing kernels.
#include "tcgen05.cuh"

#include <cfloat>

using namespace pae;

namespace {

using pae_tcgen05::mbar_expect_tx;
using pae_tcgen05::mbar_init;
using pae_tcgen05::mbar_try_wait;
using pae_tcgen05::encode_tiled;
using pae_tcgen05::EncodeTiled;

constexpr int ROWS = 16;            // weight rows per warp (the MMA's M)
constexpr int CHUNK = 64;           // of K per stage
constexpr int A_BYTES = ROWS * CHUNK * 2;      // 2 KB
constexpr uint32_t WAIT_LIMIT = 1u << 21;      // polls of a stage's mbarrier before a warp gives up
constexpr uint32_t SELFTEST_WAIT_LIMIT = 1u << 12;
constexpr int GAVE_UP = 8;          // the error word's code of a warp that gave up
constexpr int SMEM_LIMIT = 227 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ void mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One copy of `box_rows` rows x BOXES neighbouring chunks of 64 of K: the matrix is described to
// the TMA unit as [K / 64][rows][64], so that a box of (64, box_rows, BOXES) lands as BOXES tiles
// of box_rows x 128 bytes, each swizzled by itself. One instruction per stage and operand
// instead of one per chunk: at a kilobyte an instruction the TMA unit's instruction rate, not
// memory, set the pace of an SM.
__device__ __forceinline__ void tma_load_chunks(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row, int chunk) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(row), "r"(chunk)
      : "memory");
}

enum Kind : int { QKV = 0, RESIDUAL = 1, GATE_UP = 2 };

struct Params {
  const __nv_bfloat16* x;        // [tokens, k]
  int tokens, n, k;
  // the norm whose output x stands for (NORMED kernels)
  const float* norm_weight;      // [k]
  float eps;
  // RESIDUAL
  const __nv_bfloat16* residual; // [tokens, n] or null
  __nv_bfloat16* out;            // RESIDUAL: [tokens, n]; GATE_UP: [tokens, n / 2]; QKV: [tokens, n]
  // QKV
  const float* bias;             // [n] or null
  const float* rotary;           // [tokens, d]: cosines then sines, or null
  const int* slots;              // [tokens] or null
  __nv_bfloat16* keys;           // [pages, kv_heads, page_size, d]
  __nv_bfloat16* values;
  int heads, kv_heads, d, page_size;
  int* error;                    // the device's error word
  int skip_warp, skip_group;     // SELFTEST: the stage that is announced and never asked for
};

// 16-byte chunk c of row r of a [rows x 64] bfloat16 tile lives at chunk c ^ (r & 7) (TMA's
// 128-byte swizzle): the eight rows that an ldmatrix reads fall into different banks.
__device__ __forceinline__ int tile_offset(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// The first weight row of the lower (r = 0) and the upper (r = 8) eight MMA rows of warp-tile `tile`.
template <int KIND>
__device__ __forceinline__ int weight_row(const Params& p, int tile, int r) {
  if (KIND == QKV) {
    const int half = p.d >> 1, per_head = half >> 3;           // warp-tiles per head
    const int head = tile / per_head, j0 = (tile - head * per_head) * 8;
    return head * p.d + (r < 8 ? j0 : half + j0);
  }
  if (KIND == GATE_UP) {
    // rows alternate in blocks of 16 gate, 16 up; tile t holds gate rows 8t..8t+7 of the intermediate size
    const int j = tile * 8;
    return (j >> 4) * 32 + (j & 15) + (r < 8 ? 0 : 16);
  }
  return tile * ROWS + r;
}

// The normed operand in shared memory: k-step s (16 of K) of token tile n is 32 lanes x 8 bytes,
// the lane's b0 and b1 of the MMA; a step's blocks start 8 bytes further than a multiple of their
// size, so that the block's prologue, whose lanes write neighbouring steps, meets no bank twice.
template <int NT8>
__device__ __forceinline__ int operand_offset(int step, int n, int lane) { return ((step * NT8 + n) * 32 + lane) * 8 + step * 8; }
template <int NT8>
__host__ __device__ constexpr size_t operand_bytes(int k) { return (size_t)(k / 16) * (NT8 * 256 + 8); }

// NT8: n8 tiles of tokens (tokens <= 8 NT8). WARPS: warps per block. SPLIT: the block's warps
// share K out (one warp-tile per block) or each has a warp-tile of its own and the full K.
// NORMED: x is the input of an RMSNorm whose output the product takes.
template <int KIND, int NT8, int WARPS, bool SPLIT, int STAGES, int BOXES, bool NORMED, bool SELFTEST = false>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x, const Params p) {
  dependent_launch_trigger();
  extern __shared__ uint8_t smem_raw[];
  constexpr int TOKENS = 8 * NT8;
  constexpr int B_BYTES = NORMED ? 0 : TOKENS * CHUNK * 2;
  constexpr int BOX_BYTES = A_BYTES + B_BYTES;          // one chunk of 64 of K: weights, then activations
  constexpr int STAGE_BYTES = BOXES * BOX_BYTES;
  constexpr int RING_BYTES = WARPS * STAGES * STAGE_BYTES;
  constexpr int EXCHANGE_BYTES = SPLIT ? WARPS * ROWS * TOKENS * 4 : 0;
  constexpr int FRONT_BYTES = RING_BYTES > EXCHANGE_BYTES ? RING_BYTES : EXCHANGE_BYTES;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + FRONT_BYTES);                      // [WARPS][STAGES]
  float* token_scale = (float*)(smem + FRONT_BYTES + WARPS * STAGES * 8);   // [TOKENS]
  uint8_t* operand = smem + FRONT_BYTES + WARPS * STAGES * 8 + 64 * 4;   // the normed operand (NORMED)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int tile = SPLIT ? (int)blockIdx.x : (int)blockIdx.x * WARPS + warp;
  const int tiles = KIND == QKV ? (p.n / p.d) * (p.d >> 4) : (KIND == GATE_UP ? p.n / 16 : (p.n + ROWS - 1) / ROWS);
  const bool live = tile < tiles;
  const int chunks = p.k / CHUNK;
  // this warp's chunks of K
  const int per_warp = SPLIT ? (chunks + WARPS - 1) / WARPS : chunks;
  const int first = SPLIT ? min(warp * per_warp, chunks) : 0;
  const int count = live ? (SPLIT ? min(per_warp, chunks - first) : chunks) : 0;
  uint8_t* mine = smem + warp * STAGES * STAGE_BYTES;
  const uint32_t mine_u32 = smem_u32(mine);
  const uint32_t bar0 = smem_u32(bars + warp * STAGES);
  const int row_lo = live ? weight_row<KIND>(p, tile, 0) : 0, row_hi = live ? weight_row<KIND>(p, tile, 8) : 0;

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // A stage holds BOXES neighbouring chunks, asked for together (a row's bytes of one stage are
  // neighbours in memory): BOXES tiles of rows row_lo.., BOXES tiles of rows row_hi.., 8 rows
  // each, then BOXES tiles of the activations. Rows beyond the matrix and chunks beyond K read as zero.
  const int groups = (count + BOXES - 1) / BOXES;
  auto fetch_weights = [&](int group) {
    const int stage = group % STAGES;
    const uint32_t bar = bar0 + stage * 8, dst = mine_u32 + stage * STAGE_BYTES;
    mbar_expect_tx(bar, STAGE_BYTES);
    if (SELFTEST && warp == p.skip_warp && group == p.skip_group) return;
    tma_load_chunks(dst, &map_w, bar, row_lo, first + group * BOXES);
    tma_load_chunks(dst + BOXES * (A_BYTES / 2), &map_w, bar, row_hi, first + group * BOXES);
  };
  auto fetch_activations = [&](int group) {
    if (NORMED) return;
    const int stage = group % STAGES;
    if (SELFTEST && warp == p.skip_warp && group == p.skip_group) return;
    tma_load_chunks(mine_u32 + stage * STAGE_BYTES + BOXES * A_BYTES, &map_x, bar0 + stage * 8, 0, first + group * BOXES);
  };

  // The first stages' weights before the wait for the kernel before; their activations after it.
  const int early = min(groups, STAGES);
  if (lane == 0)
    for (int i = 0; i < early; ++i) fetch_weights(i);
  // What the epilogue adds comes from weights (the bias) and is asked for now ...
  const bool finishes = live && (!SPLIT || warp == 0);          // this warp runs the epilogue
  float bias_lo = 0.f, bias_hi = 0.f;
  int qkv_head = 0, qkv_f = 0;
  if (KIND == QKV) {
    const int half = p.d >> 1, per_head = half >> 3;
    qkv_head = tile / per_head;
    qkv_f = (tile - qkv_head * per_head) * 8 + g;
    if (finishes && p.bias != nullptr) {
      bias_lo = p.bias[qkv_head * p.d + qkv_f];
      bias_hi = p.bias[qkv_head * p.d + half + qkv_f];
    }
  }
  // ... and so does the first pass of the norm's weight (NORMED).
  constexpr int PASS = TOKENS / WARPS > 2 ? 4 : 8;      // 16-byte units of a token's x per lane and pass
  const int units = p.k >> 3;
  float4 gamma0[PASS][2];
  if (NORMED) {
#pragma unroll
    for (int j = 0; j < PASS; ++j) {
      const int u = 32 * j + lane;
      gamma0[j][0] = gamma0[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (u < units) {
        gamma0[j][0] = *(const float4*)(p.norm_weight + u * 8);
        gamma0[j][1] = *(const float4*)(p.norm_weight + u * 8 + 4);
      }
    }
  }
  dependent_launch_wait();
  if (lane == 0)
    for (int i = 0; i < early; ++i) fetch_activations(i);
  // ... or from the step (angles and slots, the residual) and is asked for here, a trip to the
  // L2 that the main loop hides: for tokens 8 n + 2 t4 + e.
  float side_lo[NT8][2], side_hi[NT8][2];        // QKV: cosine and sine
  __nv_bfloat16 rest_lo[NT8][2], rest_hi[NT8][2];   // RESIDUAL: the residual of rows g and g + 8, converted where it is added
  int side_slot[NT8][2];
#pragma unroll
  for (int n = 0; n < NT8; ++n) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int token = 8 * n + 2 * t4 + e;
      side_lo[n][e] = KIND == QKV ? 1.f : 0.f;
      side_hi[n][e] = 0.f;
      side_slot[n][e] = -1;
      rest_lo[n][e] = rest_hi[n][e] = __float2bfloat16_rn(0.f);
      if (!finishes || token >= p.tokens) continue;
      if (KIND == QKV) {
        if (qkv_head < p.heads + p.kv_heads && p.rotary != nullptr) {
          side_lo[n][e] = p.rotary[(size_t)token * p.d + qkv_f];
          side_hi[n][e] = p.rotary[(size_t)token * p.d + (p.d >> 1) + qkv_f];
        }
        if (qkv_head >= p.heads && p.slots != nullptr) side_slot[n][e] = p.slots[token];
      } else if (KIND == RESIDUAL && p.residual != nullptr) {
        const int r0 = tile * ROWS + g;
        if (r0 < p.n) rest_lo[n][e] = p.residual[(size_t)token * p.n + r0];
        if (r0 + 8 < p.n) rest_hi[n][e] = p.residual[(size_t)token * p.n + r0 + 8];
      }
    }
  }

  if (NORMED) {
    // The block's operand: warp w takes tokens w, w + WARPS, ...; a lane 16 bytes of x at a time,
    // PASS of them per token asked for together, so that a K of up to 2,048 costs one trip to the L2.
    float sq[TOKENS / WARPS > 0 ? TOKENS / WARPS : 1] = {};
    constexpr int MINE = TOKENS / WARPS > 0 ? TOKENS / WARPS : 1;      // tokens per warp
    for (int u0 = 0; u0 < units; u0 += 32 * PASS) {
      uint4 v[MINE][PASS];
      float4 w[PASS][2];
#pragma unroll
      for (int j = 0; j < PASS; ++j) {
        const int u = u0 + 32 * j + lane;
#pragma unroll
        for (int m = 0; m < MINE; ++m) {
          const int r = warp + m * WARPS;
          v[m][j] = make_uint4(0, 0, 0, 0);
          if (u < units && r < p.tokens) v[m][j] = *(const uint4*)(p.x + (size_t)r * p.k + u * 8);
        }
        if (u0 == 0) {
          w[j][0] = gamma0[j][0];
          w[j][1] = gamma0[j][1];
        } else if (u < units) {
          w[j][0] = *(const float4*)(p.norm_weight + u * 8);
          w[j][1] = *(const float4*)(p.norm_weight + u * 8 + 4);
        }
      }
#pragma unroll
      for (int j = 0; j < PASS; ++j) {
        const int u = u0 + 32 * j + lane;
        if (u >= units) continue;
        const float ws[8] = {w[j][0].x, w[j][0].y, w[j][0].z, w[j][0].w, w[j][1].x, w[j][1].y, w[j][1].z, w[j][1].w};
#pragma unroll
        for (int m = 0; m < MINE; ++m) {
          const int r = warp + m * WARPS;
          if (r >= TOKENS) continue;
          const uint32_t in[4] = {v[m][j].x, v[m][j].y, v[m][j].z, v[m][j].w};
          // unit u = k 8u..8u+7: half u & 1 (b0 or b1) of step u >> 1; its pair t goes to lane (r & 7) * 4 + t
          uint8_t* to = operand + operand_offset<NT8>(u >> 1, r >> 3, (r & 7) * 4) + (u & 1) * 4;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)&in[t]);
            sq[m] += f.x * f.x + f.y * f.y;
            const __nv_bfloat162 scaled = __floats2bfloat162_rn(f.x * ws[2 * t], f.y * ws[2 * t + 1]);
            *(uint32_t*)(to + t * 8) = *(const uint32_t*)&scaled;
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MINE; ++m) {
      const int r = warp + m * WARPS;
      const float total = warp_sum(sq[m]);
      if (lane == 0 && r < TOKENS) token_scale[r] = rsqrtf(total / (float)p.k + p.eps);
    }
    __syncthreads();
  }

  float acc[NT8][4];
#pragma unroll
  for (int n = 0; n < NT8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  constexpr uint32_t limit = SELFTEST ? SELFTEST_WAIT_LIMIT : WAIT_LIMIT;
  bool ok = true;
  int reached = 0;                   // stages that were waited for
  for (int i = 0; i < groups; ++i) {
    const int stage = i % STAGES;
    const uint32_t bar = bar0 + stage * 8, parity = (i / STAGES) & 1;
    uint32_t polls = 0;
    while (!mbar_try_wait(bar, parity)) {
      if (++polls > limit) {
        ok = false;
        break;
      }
      if (polls > 64) __nanosleep(64);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    reached = i + 1;
    const int boxes = min(BOXES, count - i * BOXES);
#pragma unroll
    for (int b = 0; b < BOXES; ++b) {
      if (b >= boxes) break;
      const uint32_t a_tile = mine_u32 + stage * STAGE_BYTES + b * (A_BYTES / 2);
      const uint8_t* b_tile = mine + stage * STAGE_BYTES + BOXES * A_BYTES + b * B_BYTES;
      const int step0 = (first + i * BOXES + b) * (CHUNK / 16);
#pragma unroll
      for (int s = 0; s < CHUNK / 16; ++s) {
        uint32_t a[4];
        // matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
        ldmatrix_x4(a, a_tile + ((lane >> 3) & 1) * (BOXES * (A_BYTES / 2)) + tile_offset(lane & 7, s * 2 + (lane >> 4)));
#pragma unroll
        for (int n = 0; n < NT8; ++n) {
          uint32_t b0, b1;
          if (NORMED) {
            const uint2 bb = *(const uint2*)(operand + operand_offset<NT8>(step0 + s, n, lane));
            b0 = bb.x;
            b1 = bb.y;
          } else {
            // B fragment: token 8 n + g, k = 2 t4, 2 t4 + 1 (b0) and + 8 (b1) of this step
            const int row = 8 * n + g;
            b0 = *(const uint32_t*)(b_tile + tile_offset(row, s * 2) + t4 * 4);
            b1 = *(const uint32_t*)(b_tile + tile_offset(row, s * 2 + 1) + t4 * 4);
          }
          mma_16816(acc[n], a, b0, b1);
        }
      }
    }
    __syncwarp();
    if (lane == 0 && i + STAGES < groups) {
      fetch_weights(i + STAGES);
      fetch_activations(i + STAGES);
    }
  }
  if (!ok) {
    // Copies that were asked for still write into this block's shared memory: wait for them
    // (bounded, and silently), then report.
    const int asked = min(groups, reached + STAGES);
    for (int i = reached; i < asked; ++i)
      for (uint32_t t = 0; t < limit && !mbar_try_wait(bar0 + (i % STAGES) * 8, (i / STAGES) & 1); ++t) __nanosleep(64);
    if (lane == 0) atomicCAS(p.error, 0, GAVE_UP);
  }

  if (SPLIT) {
    float* shared_acc = (float*)smem;                 // [WARPS][ROWS][TOKENS], over the drained ring
    __syncthreads();                                 // every warp has read its last stage
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      // acc[n]: rows g (0, 1) and g + 8 (2, 3), tokens 8 n + 2 t4, + 1
      float* to = shared_acc + (size_t)warp * ROWS * TOKENS;
      to[g * TOKENS + 8 * n + 2 * t4] = acc[n][0];
      to[g * TOKENS + 8 * n + 2 * t4 + 1] = acc[n][1];
      to[(g + 8) * TOKENS + 8 * n + 2 * t4] = acc[n][2];
      to[(g + 8) * TOKENS + 8 * n + 2 * t4 + 1] = acc[n][3];
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      for (int w = 0; w < WARPS; ++w) {              // in the warps' order
        const float* from = shared_acc + (size_t)w * ROWS * TOKENS;
        acc[n][0] += from[g * TOKENS + 8 * n + 2 * t4];
        acc[n][1] += from[g * TOKENS + 8 * n + 2 * t4 + 1];
        acc[n][2] += from[(g + 8) * TOKENS + 8 * n + 2 * t4];
        acc[n][3] += from[(g + 8) * TOKENS + 8 * n + 2 * t4 + 1];
      }
    }
  }
  if (!live) return;

  // ---- epilogues: this thread holds rows g and g + 8 of the warp-tile for tokens 8 n + 2 t4, + 1
#pragma unroll
  for (int n = 0; n < NT8; ++n) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int token = 8 * n + 2 * t4 + e;
      if (token >= p.tokens) continue;
      const float sc = NORMED ? token_scale[token] : 1.f;
      float lo = acc[n][e] * sc, hi = acc[n][2 + e] * sc;            // rows g and g + 8
      if (KIND == QKV) {
        const int half = p.d >> 1, head = qkv_head, f = qkv_f;
        lo += bias_lo;
        hi += bias_hi;
        lo = __bfloat162float(__float2bfloat16_rn(lo));
        hi = __bfloat162float(__float2bfloat16_rn(hi));
        if (head < p.heads + p.kv_heads && p.rotary != nullptr) rotate_pair(lo, hi, side_lo[n][e], side_hi[n][e]);
        const __nv_bfloat16 lo16 = __float2bfloat16_rn(lo), hi16 = __float2bfloat16_rn(hi);
        __nv_bfloat16* q = p.out + (size_t)token * p.n + head * p.d;
        q[f] = lo16;
        q[half + f] = hi16;
        if (head >= p.heads && p.slots != nullptr) {
          const int slot = side_slot[n][e];
          if (slot >= 0 && slot_in_pool(slot, p.page_size)) {
            const int page = slot / p.page_size, offset = slot - page * p.page_size;
            const bool is_key = head < p.heads + p.kv_heads;
            const int kv_head = is_key ? head - p.heads : head - p.heads - p.kv_heads;
            __nv_bfloat16* to = (is_key ? p.keys : p.values) + (((size_t)page * p.kv_heads + kv_head) * p.page_size + offset) * p.d;
            to[f] = lo16;
            to[half + f] = hi16;
          }
        }
      } else if (KIND == GATE_UP) {
        const int j = tile * 8 + g;
        const float gate = __bfloat162float(__float2bfloat16_rn(lo)), up = __bfloat162float(__float2bfloat16_rn(hi));
        p.out[(size_t)token * (p.n >> 1) + j] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      } else {
        const int row_lo = tile * ROWS + g, row_hi = row_lo + 8;
        if (row_lo < p.n) {
          lo += __bfloat162float(rest_lo[n][e]);
          p.out[(size_t)token * p.n + row_lo] = __float2bfloat16_rn(lo);
        }
        if (row_hi < p.n) {
          hi += __bfloat162float(rest_hi[n][e]);
          p.out[(size_t)token * p.n + row_hi] = __float2bfloat16_rn(hi);
        }
      }
    }
  }
}


struct ChunkMapKey {
  const void* ptr;
  int rows, k, box_rows, boxes;
  bool operator==(const ChunkMapKey& o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows && boxes == o.boxes; }
};
struct ChunkMapKeyHash {
  size_t operator()(const ChunkMapKey& key) const {
    size_t h = (size_t)key.ptr;
    h = h * 1000003u ^ (size_t)key.rows;
    h = h * 1000003u ^ (size_t)key.k;
    h = h * 1000003u ^ (size_t)key.box_rows;
    return h * 1000003u ^ (size_t)key.boxes;
  }
};

// A [rows, k] bfloat16 row-major matrix as [k / 64][rows][64] (strides 128 bytes, k * 2 bytes,
// one element), boxes of 64 x box_rows x boxes with 128-byte swizzle, zero fill outside.
int chunk_map(CUtensorMap* out, const void* ptr, int rows, int k, int box_rows, int boxes) {
  static std::mutex mutex;
  static std::unordered_map<ChunkMapKey, CUtensorMap, ChunkMapKeyHash> cache;
  std::lock_guard<std::mutex> guard(mutex);
  const ChunkMapKey key{ptr, rows, k, box_rows, boxes};
  auto found = cache.find(key);
  if (found != cache.end()) {
    *out = found->second;
    return 0;
  }
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return fail(101, "linear_few_tokens: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[3] = {(cuuint64_t)CHUNK, (cuuint64_t)rows, (cuuint64_t)(k / CHUNK)};
  const cuuint64_t strides[2] = {(cuuint64_t)k * 2, (cuuint64_t)CHUNK * 2};
  const cuuint32_t box[3] = {(cuuint32_t)CHUNK, (cuuint32_t)box_rows, (cuuint32_t)boxes};
  const cuuint32_t element_strides[3] = {1, 1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, element_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(102, "linear_few_tokens: cuTensorMapEncodeTiled failed with %d for [%d, %d]", (int)r, rows, k);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

template <int KIND, int NT8, int WARPS, bool SPLIT, int STAGES, int BOXES, bool NORMED>
constexpr size_t shared_bytes(int k) {
  constexpr size_t TOKENS = 8 * NT8;
  constexpr size_t stage = BOXES * (A_BYTES + (NORMED ? 0 : TOKENS * CHUNK * 2));
  constexpr size_t ring = (size_t)WARPS * STAGES * stage;
  constexpr size_t exchange = SPLIT ? (size_t)WARPS * ROWS * TOKENS * 4 : 0;
  return 1024 + (ring > exchange ? ring : exchange) + (size_t)WARPS * STAGES * 8 + 64 * 4 + (NORMED ? operand_bytes<NT8>(k) : 0);
}

template <int KIND, int NT8, int WARPS, bool SPLIT, int STAGES, int BOXES, bool NORMED>
int launch_one(const Params& p, const void* w, int tiles, cudaStream_t stream) {
  const size_t bytes = shared_bytes<KIND, NT8, WARPS, SPLIT, STAGES, BOXES, NORMED>(p.k);
  if (bytes > (size_t)SMEM_LIMIT) return fail(2, "linear_few_tokens: %d tokens x K = %d need %zu bytes of shared memory", p.tokens, p.k, bytes);
  // A ring that fits no K at all (the activations' chunks beside the weights' for many tokens) is not compiled.
  if constexpr (shared_bytes<KIND, NT8, WARPS, SPLIT, STAGES, BOXES, NORMED>(CHUNK) <= (size_t)SMEM_LIMIT) {
  auto kernel = gemv_kernel<KIND, NT8, WARPS, SPLIT, STAGES, BOXES, NORMED>;
  // The attribute belongs to the kernel as loaded on one device.
  static size_t configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return fail(100, "linear_few_tokens: no current device");
  if (bytes > configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err != cudaSuccess) return fail(100, "linear_few_tokens: %s", cudaGetErrorString(err));
    configured[device] = bytes;
  }
  CUtensorMap map_w, map_x;
  if (int err = chunk_map(&map_w, w, p.n, p.k, 8, BOXES)) return err;
  if (NORMED) map_x = map_w;       // not read
  else if (int err = chunk_map(&map_x, p.x, p.tokens, p.k, 8 * NT8, BOXES)) return err;
  const int blocks = SPLIT ? tiles : (tiles + WARPS - 1) / WARPS;
  launch_kernel(kernel, dim3(blocks), dim3(WARPS * 32), bytes, stream, map_w, map_x, p);
  return check_launch("linear_few_tokens");
  } else {
    return fail(2, "linear_few_tokens: no such kernel");
  }
}

// What decides the shape of a launch: warps per block, stages per warp's ring and chunks per
// stage. What counts is how many neighbouring bytes of a weight row are asked for at once (a
// stage of 4 chunks: 512), how much is on the way per SM (warps x stages x chunks x 2 KB) and how
// much of a warp's share of K the ring holds when the wait for the kernel before ends: what it
// does not hold costs further trips to memory one after the other. Measured at 8 tokens (q|k|v, o,
// gate|up and down of a 1536-wide model in a row, 28 times over, one copy per stage and operand):
// 23.4 us with 3 stages of 3 chunks, 24.0 us with 2 of 4, 24.4 us with 4 of 2 (not built: the room of 2 of 4), 27.0 us with 2 of 2;
// with one copy per chunk 25.8 us (2 of 4), 33.1 us (8 of 1), 50.2 us (4 of 1). The first in the
// order of preference whose blocks all run at once is taken (gate|up alone is fastest with 3 stages
// of 4; with 9 to 16 tokens the activations' chunks take room beside the weights' and 3 stages of 2
// fit where 3 of 3 do not), unless `pae_linear_few_tokens_configure` has named one for the kind.
struct Shape {
  int warps, stages, boxes;
};
constexpr Shape SHAPES[] = {{8, 2, 4}, {8, 2, 2}, {8, 3, 3}, {8, 3, 4}, {8, 3, 2}};
constexpr int NUM_SHAPES = sizeof(SHAPES) / sizeof(SHAPES[0]);
int g_forced[3] = {-1, -1, -1};        // index into SHAPES, or -1

template <int KIND, int NT8, bool SPLIT, bool NORMED>
size_t shape_bytes(int index, int k) {
  switch (index) {
    case 0: return shared_bytes<KIND, NT8, 8, SPLIT, 2, 4, NORMED>(k);
    case 1: return shared_bytes<KIND, NT8, 8, SPLIT, 2, 2, NORMED>(k);
    case 2: return shared_bytes<KIND, NT8, 8, SPLIT, 3, 3, NORMED>(k);
    case 4: return shared_bytes<KIND, NT8, 8, SPLIT, 3, 2, NORMED>(k);
    default: return shared_bytes<KIND, NT8, 8, SPLIT, 3, 4, NORMED>(k);
  }
}

int sm_count() {
  static int count = [] {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) value = 0;
    return value > 0 ? value : 148;
  }();
  return count;
}

// Blocks of 256 threads and `bytes` of shared memory that an SM holds (228 KB, 1 KB of them taken per block).
int blocks_per_sm(size_t bytes) {
  const int by_memory = (int)((size_t)228 * 1024 / (bytes + 1024));
  return by_memory < 8 ? by_memory : 8;
}

// The shape of a launch of `blocks` blocks: the first whose blocks all run at once, else the
// first that fits shared memory, else -1. `at_once` tells which it was. (A second wave of blocks
// starts with empty rings and, where the input is normed, builds the operand again: the
// tcgen05 products are faster then.)
template <int KIND, int NT8, bool SPLIT, bool NORMED>
int pick_shape(int k, long blocks, bool* at_once = nullptr) {
  if (at_once != nullptr) *at_once = false;
  int fits = -1;
  // indices into SHAPES in the order of preference
  static constexpr int NORMED_ORDER[NUM_SHAPES] = {3, 0, 2, 4, 1}, PLAIN_ORDER[NUM_SHAPES] = {2, 0, 4, 1, 3};
  for (int at = 0; at < NUM_SHAPES; ++at) {
    const int i = NORMED ? NORMED_ORDER[at] : PLAIN_ORDER[at];
    if (g_forced[KIND] >= 0 && i != g_forced[KIND]) continue;
    const size_t bytes = shape_bytes<KIND, NT8, SPLIT, NORMED>(i, k);
    if (bytes > (size_t)SMEM_LIMIT) continue;
    if (fits < 0) fits = i;
    if (blocks <= (long)sm_count() * blocks_per_sm(bytes)) {
      if (at_once != nullptr) *at_once = true;
      return i;
    }
  }
  return fits;
}

template <int KIND, int NT8, bool SPLIT, bool NORMED>
int launch_shape(const Params& p, const void* w, int tiles, cudaStream_t stream) {
  switch (pick_shape<KIND, NT8, SPLIT, NORMED>(p.k, SPLIT ? tiles : (tiles + 7) / 8)) {
    case 0: return launch_one<KIND, NT8, 8, SPLIT, 2, 4, NORMED>(p, w, tiles, stream);
    case 1: return launch_one<KIND, NT8, 8, SPLIT, 2, 2, NORMED>(p, w, tiles, stream);
    case 2: return launch_one<KIND, NT8, 8, SPLIT, 3, 3, NORMED>(p, w, tiles, stream);
    case 3: return launch_one<KIND, NT8, 8, SPLIT, 3, 4, NORMED>(p, w, tiles, stream);
    case 4: return launch_one<KIND, NT8, 8, SPLIT, 3, 2, NORMED>(p, w, tiles, stream);
  }
  return fail(2, "linear_few_tokens: %d tokens x K = %d do not fit shared memory", p.tokens, p.k);
}

template <int KIND, bool SPLIT>
int launch_tokens(const Params& p, const void* w, int tiles, cudaStream_t stream) {
  const bool normed = p.norm_weight != nullptr;
  if (p.tokens <= 8) return normed ? launch_shape<KIND, 1, SPLIT, true>(p, w, tiles, stream) : launch_shape<KIND, 1, SPLIT, false>(p, w, tiles, stream);
  if (p.tokens <= 16) return normed ? launch_shape<KIND, 2, SPLIT, true>(p, w, tiles, stream) : launch_shape<KIND, 2, SPLIT, false>(p, w, tiles, stream);
  return normed ? launch_shape<KIND, 3, SPLIT, true>(p, w, tiles, stream) : launch_shape<KIND, 3, SPLIT, false>(p, w, tiles, stream);
}

constexpr int MAX_TOKENS = 24;

int check_common(const char* what, const void* w, const void* x, const void* norm_weight, const int* error, int tokens, int n, int k) {
  if (tokens < 1 || tokens > MAX_TOKENS) return fail(2, "%s: %d tokens (1 to %d)", what, tokens, MAX_TOKENS);
  if (k < CHUNK || k % CHUNK) return fail(2, "%s: K = %d is not a multiple of 64", what, k);
  if (n < 1) return fail(2, "%s: %d rows", what, n);
  if (((uintptr_t)w | (uintptr_t)x | (uintptr_t)norm_weight) & 15) return fail(2, "%s: an operand does not start on a 16-byte boundary", what);
  if (error == nullptr) return fail(2, "%s: no error word", what);
  return 0;
}

}  // namespace

template <int KIND, bool SPLIT>
int answer(int tokens, long blocks, int k, int normed) {
  bool at_once = false;
  int shape;
  if (tokens <= 8) shape = normed ? pick_shape<KIND, 1, SPLIT, true>(k, blocks, &at_once) : pick_shape<KIND, 1, SPLIT, false>(k, blocks, &at_once);
  else if (tokens <= 16) shape = normed ? pick_shape<KIND, 2, SPLIT, true>(k, blocks, &at_once) : pick_shape<KIND, 2, SPLIT, false>(k, blocks, &at_once);
  else shape = normed ? pick_shape<KIND, 3, SPLIT, true>(k, blocks, &at_once) : pick_shape<KIND, 3, SPLIT, false>(k, blocks, &at_once);
  return shape < 0 ? 0 : (at_once ? 2 : 1);
}

// Whether these kernels take a product of `kind` (0: q|k|v, 1: o and down, 2: gate|up) with
// `n` weight rows: 0 no (the shape, or the shared memory that the rings and a normed operand
// need), 1 yes, 2 yes and all of its blocks run at once, which is where it is faster than a
// tcgen05 product and the kernel that sums its splits. `normed`: with the RMSNorm of its input folded in.
PAE_EXPORT int pae_linear_few_tokens_supports(int kind, int tokens, int n, int k, int normed) {
  if (tokens < 1 || tokens > MAX_TOKENS || k < CHUNK || k % CHUNK || n < 1) return 0;
  const long tiles = (n + ROWS - 1) / ROWS;
  if (kind == QKV) return answer<QKV, true>(tokens, tiles, k, normed);
  if (kind == RESIDUAL) return answer<RESIDUAL, true>(tokens, tiles, k, normed);
  if (kind == GATE_UP) return answer<GATE_UP, false>(tokens, (tiles + 7) / 8, k, normed);
  return 0;
}

// Names the shape (warps per block, ring stages per warp, chunks of 64 of K per stage) of the
// launches of one kind (0: q|k|v, 1: o and down, 2: gate|up), which must be one of the built
// ones; warps = 0 gives the choice back to the library.
PAE_EXPORT int pae_linear_few_tokens_configure(int kind, int warps, int stages, int boxes) {
  if (kind < 0 || kind > 2) return fail(2, "linear_few_tokens_configure: kind %d", kind);
  if (warps == 0) {
    g_forced[kind] = -1;
    return 0;
  }
  for (int i = 0; i < NUM_SHAPES; ++i)
    if (SHAPES[i].warps == warps && SHAPES[i].stages == stages && SHAPES[i].boxes == boxes) {
      g_forced[kind] = i;
      return 0;
    }
  return fail(2, "linear_few_tokens_configure: no kernel of %d warps, %d stages, %d chunks a stage", warps, stages, boxes);
}

// out[token, n] = x (or RMSNorm(x) with `norm_weight`, eps) . w[n, k]^T (+ residual[token, n]), bfloat16.
PAE_EXPORT int pae_linear_few_tokens(void* out, const void* x, const void* w, const void* residual, const float* norm_weight,
                                     float eps, int tokens, int n, int k, int* error, void* stream) {
  if (int err = check_common("linear_few_tokens", w, x, norm_weight, error, tokens, n, k)) return err;
  Params p{};
  p.x = (const __nv_bfloat16*)x;
  p.tokens = tokens;
  p.n = n;
  p.k = k;
  p.norm_weight = norm_weight;
  p.eps = eps;
  p.residual = (const __nv_bfloat16*)residual;
  p.out = (__nv_bfloat16*)out;
  p.error = error;
  return launch_tokens<RESIDUAL, true>(p, w, (n + ROWS - 1) / ROWS, (cudaStream_t)stream);
}

// out[token, inter] = SiLU(g) * u with g, u = RMSNorm(x) . (gate, up rows of w)^T, each rounded to
// bfloat16 first; w [2 inter, k] with rows alternating in blocks of 16 gate, 16 up.
PAE_EXPORT int pae_linear_swiglu_few_tokens(void* out, const void* x, const void* w, const float* norm_weight, float eps,
                                            int tokens, int two_inter, int k, int* error, void* stream) {
  if (int err = check_common("linear_swiglu_few_tokens", w, x, norm_weight, error, tokens, two_inter, k)) return err;
  if (two_inter % 32) return fail(2, "linear_swiglu_few_tokens: %d rows are not blocks of 16 gate and 16 up rows", two_inter);
  Params p{};
  p.x = (const __nv_bfloat16*)x;
  p.tokens = tokens;
  p.n = two_inter;
  p.k = k;
  p.norm_weight = norm_weight;
  p.eps = eps;
  p.out = (__nv_bfloat16*)out;
  p.error = error;
  return launch_tokens<GATE_UP, false>(p, w, two_inter / 16, (cudaStream_t)stream);
}

// qkv[token, (heads + 2 kv_heads) d] = RMSNorm(x) . w^T + bias, q and k rotated by `rotary`
// [tokens, d] (cosines, then sines; or null), k and v also written to their pages at `slots`.
PAE_EXPORT int pae_qkv_few_tokens(void* qkv, const void* x, const void* w, const float* bias, const float* norm_weight,
                                  float eps, const float* rotary, const int* slots, void* keys, void* values, int tokens,
                                  int heads, int kv_heads, int d, int page_size, int k, int* error, void* stream) {
  const int n = (heads + 2 * kv_heads) * d;
  if (int err = check_common("qkv_few_tokens", w, x, norm_weight, error, tokens, n, k)) return err;
  if (d < 16 || d % 16) return fail(2, "qkv_few_tokens: head_dim %d is not a multiple of 16", d);
  if (slots != nullptr && (keys == nullptr || values == nullptr || page_size < 1)) return fail(2, "qkv_few_tokens: slots without pages");
  Params p{};
  p.x = (const __nv_bfloat16*)x;
  p.tokens = tokens;
  p.n = n;
  p.k = k;
  p.norm_weight = norm_weight;
  p.eps = eps;
  p.out = (__nv_bfloat16*)qkv;
  p.bias = bias;
  p.rotary = rotary;
  p.slots = slots;
  p.keys = (__nv_bfloat16*)keys;
  p.values = (__nv_bfloat16*)values;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.d = d;
  p.page_size = page_size;
  p.error = error;
  return launch_tokens<QKV, true>(p, w, (heads + 2 * kv_heads) * (d / 16), (cudaStream_t)stream);
}

// The give-up path, exercised without a fault: o-or-down product of up to 8 tokens in which
// warp `skip_warp` of every block announces its stage `skip_group` to the mbarrier and never asks
// for it. That warp's wait runs out after a few thousand polls (not the two million of the
// product path), it waits likewise for what else it had asked for, sets the error word to 8 and the kernel
// ends by itself; `out` then means nothing.
PAE_EXPORT int pae_linear_few_tokens_selftest_giveup(void* out, const void* x, const void* w, int tokens, int n, int k,
                                                     int skip_warp, int skip_group, int* error, void* stream) {
  if (int err = check_common("linear_few_tokens_selftest_giveup", w, x, nullptr, error, tokens, n, k)) return err;
  if (tokens > 8) return fail(2, "linear_few_tokens_selftest_giveup: %d tokens (1 to 8)", tokens);
  Params p{};
  p.x = (const __nv_bfloat16*)x;
  p.tokens = tokens;
  p.n = n;
  p.k = k;
  p.out = (__nv_bfloat16*)out;
  p.error = error;
  p.skip_warp = skip_warp;
  p.skip_group = skip_group;
  constexpr size_t bytes = shared_bytes<RESIDUAL, 1, 8, true, 2, 2, false>(0);
  auto kernel = gemv_kernel<RESIDUAL, 1, 8, true, 2, 2, false, true>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) return fail(100, "linear_few_tokens_selftest_giveup: %s", cudaGetErrorString(err));
  CUtensorMap map_w, map_x;
  if (int e = chunk_map(&map_w, w, n, k, 8, 2)) return e;
  if (int e = chunk_map(&map_x, x, tokens, k, 8, 2)) return e;
  launch_kernel(kernel, dim3((n + ROWS - 1) / ROWS), dim3(256), bytes, (cudaStream_t)stream, map_w, map_x, p);
  return check_launch("linear_few_tokens_selftest_giveup");
}

PAE_DEFINE_LAST_ERROR()

// Attention of prompt portions over the paged cache on the fifth-generation tensor cores:
// both products of attention are tcgen05.mma with accumulators in tensor memory, keys and
// values come page by page through TMA, and the softmax runs in plain threads beside them.
//
// A block owns 128 consecutive query tokens of one request and one query head, and walks
// that request's keys 128 at a time:
//
//   warp 0      TMA: the query tile once; per key tile the pages of K and of V (one box of
//               page_size rows x 64 columns per page and half of the head dimension), two
//               stages deep. Pages are found through the block table; nothing is gathered.
//   warp 1      MMA: S = Q . K^T into one of two score buffers in tensor memory (so the
//               scores of the next tile are computed while the softmax works on this one),
//               then O_tile = P . V, into one of two product buffers, once the probabilities
//               are in one of two buffers in shared memory. V is used as it lies in the
//               cache (head dimension contiguous): an MN-major operand.
//   warps 2-9   softmax: two threads share query row r (half of a tile's keys and half of
//               the output's dimensions each). A thread reads its scores from tensor memory
//               twice (maximum; then exponentials, sum and the bfloat16 probabilities
//               written to shared memory in the operand's swizzled layout). The product of
//               a tile is folded into the running output in registers one tile late,
//               out = out * 2^(old max - new max) + O_tile, so the tensor core computes it
//               while the threads take the next tile's exponentials. No shuffles.
//
// The rule of the reference (engine/attention.py:581-586) is evaluated per score on tiles
// that touch the diagonal, a window's edge or the request's end; tiles that lie wholly
// inside need no mask. Scores are scaled in float32; probabilities are rounded to bfloat16
// for the second product. Every mbarrier wait is bounded and reports through `error`.
//
// When a launch has few blocks (a short portion of a prompt over a long context), a query
// tile's keys are shared out over a thread-block cluster: every block of the cluster takes a
// run of key tiles, the blocks behind the first leave their rows' maxima, sums and outputs in
// their own shared memory, and the first merges them through distributed shared memory
// between two barriers of the cluster.
//
// Sizes: head_dim 64 or 128; page sizes 16, 32, 64 or 128; any number of heads and groups.
// Requests that bring a single token are left to the decode kernel.
#include <cuda.h>

#include <cfloat>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

using namespace pae;

namespace {

constexpr int BQ = 128;             // query rows per block
constexpr int BKEYS = 128;          // keys per tile
constexpr int THREADS = 320;         // TMA warp, MMA warp, eight softmax warps (two threads per query row)
constexpr int SOFTMAX_THREADS = 256;
constexpr uint32_t WAIT_LIMIT = 1u << 21;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  __nv_bfloat16* out;               // [tokens, heads, D]
  const int* block_table;
  const int* q_start;
  const int* q_pos0;
  const int* kv_len;
  int table_width, heads, kv_heads, page_size, window, skip_single;
  const int* work_index;  // the requests that this launch works on, one per grid z (null: request z)
  float scale_log2;
  int* error;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error, int code) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (i > 64) __nanosleep(64);
  }
  *abort_flag = 1;
  atomicCAS(error, 0, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t holder, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 consecutive float32 columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_load32(uint32_t address, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The cluster's barrier (every thread of every block of the cluster arrives and waits), this
// block's place in its cluster, and a float read from the shared memory of another block of it.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t n;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
  return n;
}
__device__ __forceinline__ float load_from_block(uint32_t address, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(address), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// K-major operand tile with 128-byte swizzle (rows of 64 bfloat16, groups of 8 rows 1024 bytes apart).
__device__ __forceinline__ uint64_t k_major_descriptor(uint32_t address) {
  uint64_t d = 0;
  d |= (uint64_t)((address & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand with 128-byte swizzle: a 128-byte row holds 64 consecutive MN elements of
// one K index; 8 consecutive K indices are 8 rows (1024 bytes, the stride byte offset); the
// next 64 MN elements lie `mn_group_bytes` further (the leading byte offset).
__device__ __forceinline__ uint64_t mn_major_descriptor(uint32_t address, uint32_t mn_group_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((address & 0x3FFFFu) >> 4);
  d |= (uint64_t)((mn_group_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// float32 accumulator, bfloat16 operands, A K-major; B K-major or MN-major (bit 16).
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

template <int D>
struct Layout {
  static constexpr int HALVES = D / 64;                    // 64-column k-blocks of the head dimension
  static constexpr int HALF_TILE_BYTES = 128 * 64 * 2;     // 128 rows x 64 bfloat16 = 16 KB
  static constexpr int Q_BYTES = HALVES * HALF_TILE_BYTES;
  static constexpr int KV_BYTES = HALVES * HALF_TILE_BYTES;   // one stage of K, or of V
  static constexpr int P_BYTES = 2 * HALF_TILE_BYTES;         // 128 rows x 128 keys, one of two buffers
  static constexpr int Q_OFFSET = 0;
  static constexpr int K_OFFSET = Q_BYTES;                    // two stages
  static constexpr int V_OFFSET = K_OFFSET + 2 * KV_BYTES;
  static constexpr int P_OFFSET = V_OFFSET + 2 * KV_BYTES;
  static constexpr int BAR_OFFSET = P_OFFSET + 2 * P_BYTES;
  static constexpr int EXCHANGE_OFFSET = BAR_OFFSET + 256;    // [2][128] floats that the two threads of a row swap
  static constexpr size_t SMEM_BYTES = (size_t)EXCHANGE_OFFSET + 1024 /* exchange */ + 1024 /* alignment */;
  static constexpr int S_COLUMNS = 128;                       // per score buffer
  static constexpr int O_COLUMN = 2 * S_COLUMNS;              // two tiles' products behind the two score buffers
  static constexpr int TMEM_COLUMNS = 512;
  static_assert(O_COLUMN + 2 * D <= TMEM_COLUMNS, "two score buffers and two products must fit tensor memory");
  static_assert(SMEM_BYTES <= 227 * 1024, "the block's shared memory");
};

enum Bar : int { Q_FULL = 0, K_FULL = 1, V_FULL = 3, K_EMPTY = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11, P_READY = 13, O_FULL = 15, O_EMPTY = 17, X_READY = 19, NUM_BARS = 20 };

template <int D, bool SPLIT>
__global__ void __launch_bounds__(THREADS) prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                  const __grid_constant__ CUtensorMap map_k,
                                                                  const __grid_constant__ CUtensorMap map_v, const Params p) {
  using L = Layout<D>;
  dependent_launch_trigger();
  if (threadIdx.x == 0) {         // the descriptors do not depend on the kernel before: fetch them early
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  extern __shared__ uint8_t raw_smem[];
  const uint32_t raw = smem_u32(raw_smem);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* generic_base = raw_smem + (base - raw);
  const uint32_t bars = base + L::BAR_OFFSET;
  volatile uint32_t* tmem_holder = (volatile uint32_t*)(generic_base + L::BAR_OFFSET + 8 * NUM_BARS);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  auto bar = [&](int which, int i = 0) { return bars + 8u * (which + i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(K_FULL, i), 1);
      mbar_init(bar(V_FULL, i), 1);
      mbar_init(bar(K_EMPTY, i), 1);
      mbar_init(bar(V_EMPTY, i), 1);
      mbar_init(bar(S_FULL, i), 1);
      mbar_init(bar(S_EMPTY, i), SOFTMAX_THREADS);
      mbar_init(bar(P_READY, i), SOFTMAX_THREADS);
      mbar_init(bar(O_FULL, i), 1);
      mbar_init(bar(O_EMPTY, i), SOFTMAX_THREADS);
    }
    mbar_init(bar(X_READY), SOFTMAX_THREADS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_holder), L::TMEM_COLUMNS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // ---- what this block works on (the same in every role) -------------------------------
  // The step's integers (starts, positions, lengths, block tables) were on the device before
  // the step's first kernel began: they are read before the wait for the kernel before this
  // one, whose output (q, and this step's keys and values) is not touched until after it.
  // A cluster of `ranks` blocks shares one query tile of one head: each takes a run of its key
  // tiles, and the first block folds the others' outputs into its own at the end.
  const int ranks = SPLIT ? (int)cluster_size() : 1, rank = SPLIT ? (int)cluster_rank() : 0;
  const int h = blockIdx.x / ranks, b = p.work_index != nullptr ? p.work_index[blockIdx.z] : (int)blockIdx.z;
  const int first_token = p.q_start[b];
  const int q_count = p.q_start[b + 1] - first_token;
  const int q_tiles = (q_count + BQ - 1) / BQ;
  // Late tiles see the most keys: they go first in every head (the head is the fastest grid
  // index, so the first wave holds the longest blocks of all heads), the short early ones
  // fill in behind them.
  const int tile = q_tiles - 1 - (int)blockIdx.y;
  const bool active = tile >= 0 && !(p.skip_single && q_count == 1);
  const int rows = active ? min(BQ, q_count - tile * BQ) : 0;
  const int pos0 = p.q_pos0[b] + tile * BQ;
  const int kv_end = active ? min(p.kv_len[b], pos0 + rows) : 0;
  const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int all_tiles = active ? (kv_end - (first_key / p.page_size) * p.page_size + BKEYS - 1) / BKEYS : 0;
  const int tiles_per_rank = (all_tiles + ranks - 1) / ranks;
  const int first_tile = min(rank * tiles_per_rank, all_tiles);
  const int n_tiles = min(tiles_per_rank, all_tiles - first_tile);          // this block's
  const int kv_begin = (first_key / p.page_size) * p.page_size + first_tile * BKEYS;
  const bool working = n_tiles > 0;
  const int g = h / (p.heads / p.kv_heads);

  // What the softmax threads carry out of their loop (the other warps leave it alone).
  constexpr int HALF_D = D / 2;
  const int quadrant = warp & 3;
  const int side = warp >= 2 ? (warp - 2) >> 2 : 0;         // which half of the keys and of the dimensions
  const int r = quadrant * 32 + lane;                       // row of the tile, lane of tensor memory
  float acc[HALF_D];
  float row_max = -FLT_MAX, row_sum = 0.f;
  bool ok = true;
  // The producer's lane i brings page i of a tile: the first tile's table entries, before the wait.
  const int last_page = working ? (kv_end - 1) / p.page_size : 0;    // the last page that holds a visible key
  int first_page = 0;
  if (warp == 0 && working && lane < BKEYS / p.page_size)
    first_page = checked_page(p.block_table[(size_t)b * p.table_width + checked_table_index(min(kv_begin / p.page_size + lane, last_page), p.table_width)]);
  dependent_launch_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // Lane i brings page i of a tile (its block-table entry and its boxes), so the table
    // look-ups of a tile are one round trip, not one per page. Lane 0 posts the byte counts
    // before any lane issues a copy.
    if (working) {
      if (lane == 0) {
        mbar_expect_tx(bar(Q_FULL), L::Q_BYTES);
#pragma unroll
        for (int half = 0; half < L::HALVES; ++half)
          tma_load_2d(base + L::Q_OFFSET + half * L::HALF_TILE_BYTES, &map_q, bar(Q_FULL), h * D + half * 64,
                      first_token + tile * BQ);
      }
      const int* table = p.block_table + (size_t)b * p.table_width;
      const int pages_per_tile = BKEYS / p.page_size;
      const int page_rows_bytes = p.page_size * 128;
      const bool mine = lane < pages_per_tile;
      // A page past the last visible key may not exist: its rows are masked, so any page of
      // the request will do; the last visible one is taken.
      int page = first_page;
      int issued = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1;
        int next_page = 0;
        if (mine && t + 1 < n_tiles)
          next_page = checked_page(table[checked_table_index(min((kv_begin + (t + 1) * BKEYS) / p.page_size + lane, last_page), p.table_width)]);
        if (t >= 2) {
          if (lane == 0) ok = mbar_wait(bar(K_EMPTY, st), ((t >> 1) - 1) & 1, abort_flag, p.error, 1);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (lane == 0) mbar_expect_tx(bar(K_FULL, st), L::KV_BYTES);
        __syncwarp();
        const int row = (page * p.kv_heads + g) * p.page_size;
        const uint32_t dst = st * L::KV_BYTES + lane * page_rows_bytes;
        if (mine) {
#pragma unroll
          for (int half = 0; half < L::HALVES; ++half)
            tma_load_2d(base + L::K_OFFSET + dst + half * L::HALF_TILE_BYTES, &map_k, bar(K_FULL, st), half * 64, row);
        }
        if (t >= 2) {
          if (lane == 0) ok = mbar_wait(bar(V_EMPTY, st), ((t >> 1) - 1) & 1, abort_flag, p.error, 10);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (lane == 0) mbar_expect_tx(bar(V_FULL, st), L::KV_BYTES);
        __syncwarp();
        if (mine) {
#pragma unroll
          for (int half = 0; half < L::HALVES; ++half)
            tma_load_2d(base + L::V_OFFSET + dst + half * L::HALF_TILE_BYTES, &map_v, bar(V_FULL, st), half * 64, row);
        }
        page = next_page;
        issued = t + 1;
      }
      if (lane == 0 && *abort_flag) {
        for (int t = max(0, issued - 2); t < issued; ++t) {
          for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar(K_FULL, t & 1), (t >> 1) & 1); ++w) __nanosleep(64);
          for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar(V_FULL, t & 1), (t >> 1) & 1); ++w) __nanosleep(64);
        }
        for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar(Q_FULL), 0); ++w) __nanosleep(64);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && working) {
      constexpr uint32_t idesc_s = instruction_descriptor(BQ, BKEYS, false);
      constexpr uint32_t idesc_o = instruction_descriptor(BQ, D, true);
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.error, 2);
      auto issue_scores = [&](int t) {
        const int st = t & 1;
        ok = ok && mbar_wait(bar(K_FULL, st), (t >> 1) & 1, abort_flag, p.error, 3);
        if (t >= 2) ok = ok && mbar_wait(bar(S_EMPTY, st), ((t >> 1) - 1) & 1, abort_flag, p.error, 4);
        if (!ok) return;
        tcgen05_fence_after();
        const uint32_t q_addr = base + L::Q_OFFSET, k_addr = base + L::K_OFFSET + st * L::KV_BYTES;
#pragma unroll
        for (int half = 0; half < L::HALVES; ++half)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + st * L::S_COLUMNS, k_major_descriptor(q_addr + half * L::HALF_TILE_BYTES + k * 32),
                      k_major_descriptor(k_addr + half * L::HALF_TILE_BYTES + k * 32), idesc_s, (half > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(bar(S_FULL, st));
        tcgen05_commit(bar(K_EMPTY, st));       // the K stage is free once these MMAs have read it
      };
      if (n_tiles > 0) issue_scores(0);
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) issue_scores(t + 1);
        const int st = t & 1;
        ok = ok && mbar_wait(bar(V_FULL, st), (t >> 1) & 1, abort_flag, p.error, 5);
        ok = ok && mbar_wait(bar(P_READY, st), (t >> 1) & 1, abort_flag, p.error, 6);
        if (t >= 2) ok = ok && mbar_wait(bar(O_EMPTY, st), ((t >> 1) - 1) & 1, abort_flag, p.error, 7);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t p_addr = base + L::P_OFFSET + st * L::P_BYTES, v_addr = base + L::V_OFFSET + st * L::KV_BYTES;
#pragma unroll
        for (int k = 0; k < BKEYS / 16; ++k)     // 16 keys a step: two groups of 8 rows of V
          umma_bf16(tmem_base + L::O_COLUMN + st * D, k_major_descriptor(p_addr + (k >> 2) * L::HALF_TILE_BYTES + (k & 3) * 32),
                    mn_major_descriptor(v_addr + k * 2048, L::HALF_TILE_BYTES), idesc_o, k > 0 ? 1u : 0u);
        tcgen05_commit(bar(O_FULL, st));
        tcgen05_commit(bar(V_EMPTY, st));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, two threads per row
    // The two warps that may read a quarter of tensor memory's lanes (warp id modulo 4) share
    // its 32 rows: one takes keys 0-63 of a tile and the first half of the output's
    // dimensions, the other keys 64-127 and the second half. They swap their maxima through
    // shared memory once per tile and their sums once at the end.
    //
    // P and a tile's product P.V have two buffers each, and a tile's product is added to the
    // output one tile late: after the probabilities of tile t are handed over, the threads add
    // the product of tile t-1, which the tensor core finished while they were taking
    // exponentials. So the product of one tile runs under the softmax of the next, and the
    // threads wait for neither.
    const uint32_t lane_base = tmem_base + ((uint32_t)(quadrant * 32) << 16);
    const int my_pos = pos0 + r;
    float* exchange = (float*)(generic_base + L::EXCHANGE_OFFSET);
    constexpr int HALF_KEYS = BKEYS / 2;
#pragma unroll
    for (int i = 0; i < HALF_D; ++i) acc[i] = 0.f;
    // acc = acc * scale + the product of tile u (scale: what tile u's maximum did to the reference).
    auto add_product = [&](int u, float scale) {
      const int su = u & 1;
      ok = ok && mbar_wait(bar(O_FULL, su), (u >> 1) & 1, abort_flag, p.error, 9);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      tcgen05_fence_after();
#pragma unroll
      for (int c = 0; c < HALF_D; c += 32) {
        float o[32];
        tmem_load32(lane_base + L::O_COLUMN + su * D + side * HALF_D + c, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c + i] = acc[c + i] * scale + o[i];
      }
      tcgen05_fence_before();
      mbar_arrive(bar(O_EMPTY, su));
    };
    float owed_scale = 0.f;       // goes with the product that is not added yet
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t & 1;
      const int key0 = kv_begin + t * BKEYS;
      ok = ok && mbar_wait(bar(S_FULL, st), (t >> 1) & 1, abort_flag, p.error, 8);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      // The whole tile is visible to every row of the block: no mask. Otherwise a row sees the
      // keys lo..hi of the request (nothing when the row is past the request's tokens).
      const bool unmasked = key0 + BKEYS - 1 <= pos0 && key0 + BKEYS <= kv_end && key0 >= first_key &&
                            (p.window <= 0 || pos0 + rows - 1 - key0 < p.window);
      const int hi = r < rows ? min(my_pos, kv_end - 1) - key0 : -1;          // relative to the tile
      const int lo = (p.window > 0 ? max(first_key, my_pos - p.window + 1) : first_key) - key0;
      float m4[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};
#pragma unroll
      for (int c = side * HALF_KEYS; c < side * HALF_KEYS + HALF_KEYS; c += 32) {
        float s[32];
        tmem_load32(lane_base + st * L::S_COLUMNS + c, s);
        if (unmasked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], s[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = c + i;
            m4[i & 3] = fmaxf(m4[i & 3], (key >= lo && key <= hi) ? s[i] : -FLT_MAX);
          }
        }
      }
      float tile_max = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      exchange[side * 128 + r] = tile_max;
      mbar_arrive(bar(X_READY));                                // all softmax threads have written theirs
      ok = mbar_wait(bar(X_READY), t & 1, abort_flag, p.error, 11);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tile_max = fmaxf(tile_max, exchange[(side ^ 1) * 128 + r]);
      if (tile_max != -FLT_MAX) tile_max *= p.scale_log2;        // the scale is positive: max(s) scales with it
      const float new_max = fmaxf(row_max, tile_max);
      const float rescale = row_max == -FLT_MAX ? 0.f : fast_exp2(row_max - new_max);
      row_max = new_max;
      // exp2(s * scale - max) as one fused multiply-add and one ex2; a row that has seen no key
      // yet keeps max = -FLT_MAX and every probability 0.
      const float offset = new_max == -FLT_MAX ? 0.f : -new_max;
      const float factor = new_max == -FLT_MAX ? 0.f : p.scale_log2;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* p_row = generic_base + L::P_OFFSET + st * L::P_BYTES + r * 128;
#pragma unroll
      for (int c = side * HALF_KEYS; c < side * HALF_KEYS + HALF_KEYS; c += 32) {
        float s[32];
        tmem_load32(lane_base + st * L::S_COLUMNS + c, s);
        if (unmasked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s[i] = fast_exp2(fmaf(s[i], factor, offset));
            sum4[i & 3] += s[i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = c + i;
            const float e = fast_exp2(fmaf(s[i], factor, offset));
            s[i] = (key >= lo && key <= hi && factor != 0.f) ? e : 0.f;
            sum4[i & 3] += s[i];
          }
        }
        // 32 keys = four 16-byte chunks of this row in the k-block c / 64, swizzled by the row.
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 packed;
          __nv_bfloat162* h2 = (__nv_bfloat162*)&packed;
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(s[j * 8 + 2 * e], s[j * 8 + 2 * e + 1]);
          const int chunk = ((c & 63) >> 3) + j;
          *(uint4*)(p_row + (c >> 6) * L::HALF_TILE_BYTES + ((chunk ^ (r & 7)) << 4)) = packed;
        }
      }
      row_sum = row_sum * rescale + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));   // this thread's keys only
      tcgen05_fence_before();
      mbar_arrive(bar(S_EMPTY, st));                            // this thread's part of the score buffer is read
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is for the tensor core's eyes
      mbar_arrive(bar(P_READY, st));
      if (t >= 1) add_product(t - 1, owed_scale);
      if (!ok) break;
      owed_scale = rescale;
    }
    if (n_tiles > 0 && ok) add_product(n_tiles - 1, owed_scale);
    // The row's sum is the two threads' sums (both are relative to the same maximum).
    ok = __all_sync(0xffffffffu, ok);
    if (working && ok) {
      exchange[side * 128 + r] = row_sum;
      mbar_arrive(bar(X_READY));
      ok = mbar_wait(bar(X_READY), n_tiles & 1, abort_flag, p.error, 12);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) row_sum += exchange[(side ^ 1) * 128 + r];
    }
  }

  if constexpr (SPLIT) {
    // The blocks behind the first leave their rows' maxima, sums and outputs in their own
    // shared memory, where the keys and values lay (every product that read those has
    // completed: the softmax threads waited for the last one); the first block reads them
    // there once the whole cluster has arrived, and nobody leaves before it has.
    float* stage = (float*)(generic_base + L::K_OFFSET);              // [D][128]: a dimension's 128 rows side by side
    float* stage_stats = (float*)(generic_base + L::V_OFFSET);        // [2][128]: maximum, sum
    if (warp >= 2 && rank != 0) {
      const bool has = working && ok;
      if (side == 0) {
        stage_stats[r] = has ? row_max : -FLT_MAX;
        stage_stats[128 + r] = has ? row_sum : 0.f;
      }
      if (has) {
#pragma unroll
        for (int i = 0; i < HALF_D; ++i) stage[(side * HALF_D + i) * 128 + r] = acc[i];
      }
    }
    cluster_arrive();
    cluster_wait();
    if (warp >= 2 && rank == 0 && working && ok) {
      for (int other = 1; other < ranks; ++other) {
        const float their_sum = load_from_block(smem_u32(stage_stats + 128 + r), other);
        if (their_sum > 0.f) {
          const float their_max = load_from_block(smem_u32(stage_stats + r), other);
          const float both = fmaxf(row_max, their_max);
          const float mine = row_max == -FLT_MAX ? 0.f : fast_exp2(row_max - both);
          const float theirs = fast_exp2(their_max - both);
#pragma unroll
          for (int i = 0; i < HALF_D; ++i)
            acc[i] = acc[i] * mine + load_from_block(smem_u32(stage + (side * HALF_D + i) * 128 + r), other) * theirs;
          row_sum = row_sum * mine + their_sum * theirs;
          row_max = both;
        }
      }
    }
    cluster_arrive();
    cluster_wait();
  }

  if (warp >= 2 && rank == 0 && ok && r < rows) {
    const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
    __nv_bfloat16* out = p.out + ((size_t)(first_token + tile * BQ + r) * p.heads + h) * D + side * HALF_D;
#pragma unroll
    for (int c = 0; c < HALF_D; c += 8) {
      uint4 packed;
      __nv_bfloat162* h2 = (__nv_bfloat162*)&packed;
#pragma unroll
      for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(acc[c + 2 * e] * inv, acc[c + 2 * e + 1] * inv);
      *(uint4*)(out + c) = packed;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, L::TMEM_COLUMNS);
  }
}

// ---------------------------------------------------------------------------------------
// The paired form, for launches of at least two blocks per SM (long prompts, many requests or
// heads). A block walks the keys 64 at a time with one softmax thread per query row, and
// keeps O in tensor memory over all tiles instead of reading each tile's product back:
// 113 KB of shared memory, 256 columns of tensor memory and 192 threads, so two blocks share
// an SM and the softmax of one overlaps the products and the waits of the other.
//
// The reference of a row is its running maximum, but it only moves when the maximum has grown
// by more than 2^8 since it was set: probabilities then stay below 256, which float32 sums and
// the bfloat16 operand hold as well as values below 1, and the output in tensor memory (which
// must be multiplied by 2^(old - new) whenever the reference moves) is touched on a row's first
// tiles only. The sum is kept against the same reference, so the quotient is exact softmax.
// ---------------------------------------------------------------------------------------
namespace paired {

constexpr int BKEYS = 64;           // keys per tile
constexpr int THREADS = 192;        // TMA warp, MMA warp, four softmax warps (one thread per query row)
constexpr int SOFTMAX_WARPS = 4;
constexpr int KV_STAGES = 2;
constexpr float REFERENCE_SLACK = 8.f;   // a row's reference follows its maximum in steps of more than 2^8

// The same 32 columns written back (the whole warp calls it).
__device__ __forceinline__ void tmem_store32(uint32_t address, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(address), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
        "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
        "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
template <int D>
struct Layout {
  static constexpr int HALVES = D / 64;                       // 64-column k-blocks of the head dimension
  static constexpr int Q_HALF_BYTES = BQ * 128;               // 128 rows x 64 bfloat16
  static constexpr int KV_HALF_BYTES = BKEYS * 128;           // 64 rows x 64 bfloat16
  static constexpr int Q_BYTES = HALVES * Q_HALF_BYTES;
  static constexpr int KV_BYTES = HALVES * KV_HALF_BYTES;     // one stage of K, or of V
  static constexpr int P_BYTES = BQ * BKEYS * 2;              // 128 rows x 64 keys: one swizzle row each
  static constexpr int Q_OFFSET = 0;
  static constexpr int K_OFFSET = Q_BYTES;                    // two stages
  static constexpr int V_OFFSET = K_OFFSET + KV_STAGES * KV_BYTES;
  static constexpr int P_OFFSET = V_OFFSET + KV_STAGES * KV_BYTES;
  static constexpr int BAR_OFFSET = P_OFFSET + P_BYTES;
  static constexpr int USED_BYTES = BAR_OFFSET + 256;
  // 768 bytes of slack for the 1024-byte alignment of the tiles: with it two blocks of head
  // size 128 still fit on one SM. The kernel checks that the slack was enough.
  static constexpr size_t SMEM_BYTES = (size_t)USED_BYTES + 768;
  static constexpr int S_COLUMNS = BKEYS;                     // per score buffer
  static constexpr int O_COLUMN = 2 * S_COLUMNS;              // O behind the two score buffers
  static constexpr int TMEM_COLUMNS = 256;
};

enum Bar : int {
  Q_FULL = 0, O_FULL = 1, S_FULL = 2, S_EMPTY = 4, P_READY = 6, P_EMPTY = 7,
  K_FULL = 8, K_EMPTY = K_FULL + KV_STAGES, V_FULL = K_EMPTY + KV_STAGES, V_EMPTY = V_FULL + KV_STAGES, NUM_BARS = V_EMPTY + KV_STAGES
};

template <int D>
__global__ void __launch_bounds__(THREADS, 2) prefill_tcgen05_paired_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                     const __grid_constant__ CUtensorMap map_k,
                                                                     const __grid_constant__ CUtensorMap map_v, const Params p) {
  using L = Layout<D>;
  dependent_launch_trigger();
  if (threadIdx.x == 0) {         // the descriptors do not depend on the kernel before: fetch them early
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  const uint32_t raw = smem_u32(raw_smem);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* generic_base = raw_smem + (base - raw);
  const uint32_t bars = base + L::BAR_OFFSET;
  volatile uint32_t* tmem_holder = (volatile uint32_t*)(generic_base + L::BAR_OFFSET + 8 * NUM_BARS);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  auto bar = [&](int which, int i = 0) { return bars + 8u * (which + i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool fits = (base - raw) + (uint32_t)L::USED_BYTES <= (uint32_t)L::SMEM_BYTES;
  if (!fits) {                     // the alignment took more than the slack: nothing is touched
    if (threadIdx.x == 0) atomicCAS(p.error, 0, 20);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(bar(K_FULL, i), 1);
      mbar_init(bar(K_EMPTY, i), 1);
      mbar_init(bar(V_FULL, i), 1);
      mbar_init(bar(V_EMPTY, i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(S_FULL, i), 1);
      mbar_init(bar(S_EMPTY, i), SOFTMAX_WARPS);     // one arrival per warp
    }
    mbar_init(bar(P_READY), SOFTMAX_WARPS);
    mbar_init(bar(P_EMPTY), 1);                      // by tcgen05.commit: the second product has read P
    mbar_init(bar(O_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_holder), L::TMEM_COLUMNS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // ---- what this block works on (the same in every role) -------------------------------
  // The step's integers are read before the wait for the kernel before this one (they were on
  // the device before the step's first kernel began); q and this step's keys and values after it.
  const int h = blockIdx.x, b = p.work_index != nullptr ? p.work_index[blockIdx.z] : (int)blockIdx.z;
  const int first_token = p.q_start[b];
  const int q_count = p.q_start[b + 1] - first_token;
  const int q_tiles = (q_count + BQ - 1) / BQ;
  // Late tiles see the most keys: they go first in every head (the head is the fastest grid
  // index, so the first wave holds the longest blocks of all heads), the short early ones
  // fill in behind them.
  const int tile = q_tiles - 1 - (int)blockIdx.y;
  const bool active = tile >= 0 && !(p.skip_single && q_count == 1);
  const int rows = active ? min(BQ, q_count - tile * BQ) : 0;
  const int pos0 = p.q_pos0[b] + tile * BQ;
  const int kv_end = active ? min(p.kv_len[b], pos0 + rows) : 0;
  const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kv_begin = (first_key / BKEYS) * BKEYS;
  const int n_tiles = active ? (kv_end - kv_begin + BKEYS - 1) / BKEYS : 0;
  const int g = h / (p.heads / p.kv_heads);
  // The producer's lane i brings box i of a tile (a page, or the 64 rows of a larger page that
  // the tile covers): the first tile's table entries, before the wait.
  const int box_rows = min(p.page_size, BKEYS);
  const int last_page = active ? (kv_end - 1) / p.page_size : 0;     // the last page that holds a visible key
  // The first tile starts on a multiple of 64 keys, which may lie pages before the window's first
  // key; those pages may have been given back (their table entries are holes). Their keys are
  // masked, so the window's first page stands in for them.
  const int window_page = first_key / p.page_size;
  int first_page = 0;
  if (warp == 0 && active && lane < BKEYS / box_rows)
    first_page = checked_page(p.block_table[(size_t)b * p.table_width +
                                            checked_table_index(max(min((kv_begin + lane * box_rows) / p.page_size, last_page), window_page), p.table_width)]);
  dependent_launch_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // Lane i brings box i of a tile (its block-table entry and its copies), so the table
    // look-ups of a tile are one round trip, not one per page. A box is a page, or the 64
    // rows of a larger page that the tile covers. Lane 0 posts the byte counts before any
    // lane issues a copy.
    if (active) {
      if (lane == 0) {
        mbar_expect_tx(bar(Q_FULL), L::Q_BYTES);
#pragma unroll
        for (int half = 0; half < L::HALVES; ++half)
          tma_load_2d(base + L::Q_OFFSET + half * L::Q_HALF_BYTES, &map_q, bar(Q_FULL), h * D + half * 64,
                      first_token + tile * BQ);
      }
      const int* table = p.block_table + (size_t)b * p.table_width;
      const int boxes = BKEYS / box_rows;
      const bool mine = lane < boxes;
      // A page past the last visible key may not exist: its rows are masked, so any page of
      // the request will do; the last visible one is taken.
      auto box_row = [&](int t) {
        const int key = kv_begin + t * BKEYS + lane * box_rows;
        const int page = checked_page(table[checked_table_index(max(min(key / p.page_size, last_page), window_page), p.table_width)]);
        return (page * p.kv_heads + g) * p.page_size + key % p.page_size;
      };
      int row = mine ? (first_page * p.kv_heads + g) * p.page_size + (kv_begin + lane * box_rows) % p.page_size : 0;
      int issued = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles; ++t) {
        const int stage = t % KV_STAGES;
        const uint32_t round = (uint32_t)(t / KV_STAGES);
        int next_row = 0;
        if (mine && t + 1 < n_tiles) next_row = box_row(t + 1);
        if (t >= KV_STAGES) {
          if (lane == 0) ok = mbar_wait(bar(K_EMPTY, stage), (round - 1) & 1, abort_flag, p.error, 1);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (lane == 0) mbar_expect_tx(bar(K_FULL, stage), L::KV_BYTES);
        __syncwarp();
        const uint32_t dst = stage * L::KV_BYTES + lane * box_rows * 128;
        if (mine) {
#pragma unroll
          for (int half = 0; half < L::HALVES; ++half)
            tma_load_2d(base + L::K_OFFSET + dst + half * L::KV_HALF_BYTES, &map_k, bar(K_FULL, stage), half * 64, row);
        }
        if (t >= KV_STAGES) {
          if (lane == 0) ok = mbar_wait(bar(V_EMPTY, stage), (round - 1) & 1, abort_flag, p.error, 10);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (lane == 0) mbar_expect_tx(bar(V_FULL, stage), L::KV_BYTES);
        __syncwarp();
        if (mine) {
#pragma unroll
          for (int half = 0; half < L::HALVES; ++half)
            tma_load_2d(base + L::V_OFFSET + dst + half * L::KV_HALF_BYTES, &map_v, bar(V_FULL, stage), half * 64, row);
        }
        row = next_row;
        issued = t + 1;
      }
      if (lane == 0 && *abort_flag) {      // copies that were issued still write into this block's shared memory
        for (int t = max(0, issued - KV_STAGES); t < issued; ++t) {
          for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar(K_FULL, t % KV_STAGES), (t / KV_STAGES) & 1); ++w) __nanosleep(64);
          for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar(V_FULL, t % KV_STAGES), (t / KV_STAGES) & 1); ++w) __nanosleep(64);
        }
        for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar(Q_FULL), 0); ++w) __nanosleep(64);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && active) {
      constexpr uint32_t idesc_s = instruction_descriptor(BQ, BKEYS, false);
      constexpr uint32_t idesc_o = instruction_descriptor(BQ, D, true);
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.error, 2);
      auto issue_scores = [&](int t) {
        const int st = t & 1, stage = t % KV_STAGES;
        ok = ok && mbar_wait(bar(K_FULL, stage), (t / KV_STAGES) & 1, abort_flag, p.error, 3);
        if (t >= 2) ok = ok && mbar_wait(bar(S_EMPTY, st), ((t >> 1) - 1) & 1, abort_flag, p.error, 4);
        if (!ok) return;
        tcgen05_fence_after();
        const uint32_t q_addr = base + L::Q_OFFSET, k_addr = base + L::K_OFFSET + stage * L::KV_BYTES;
#pragma unroll
        for (int half = 0; half < L::HALVES; ++half)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + st * L::S_COLUMNS, k_major_descriptor(q_addr + half * L::Q_HALF_BYTES + k * 32),
                      k_major_descriptor(k_addr + half * L::KV_HALF_BYTES + k * 32), idesc_s, (half > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(bar(S_FULL, st));
        tcgen05_commit(bar(K_EMPTY, stage));    // the K stage is free once these MMAs have read it
      };
      if (n_tiles > 0) issue_scores(0);
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) issue_scores(t + 1);
        const int stage = t % KV_STAGES;
        ok = ok && mbar_wait(bar(V_FULL, stage), (t / KV_STAGES) & 1, abort_flag, p.error, 5);
        ok = ok && mbar_wait(bar(P_READY), t & 1, abort_flag, p.error, 6);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t p_addr = base + L::P_OFFSET, v_addr = base + L::V_OFFSET + stage * L::KV_BYTES;
#pragma unroll
        for (int k = 0; k < BKEYS / 16; ++k)     // 16 keys a step: two groups of 8 rows of V
          umma_bf16(tmem_base + L::O_COLUMN, k_major_descriptor(p_addr + k * 32),
                    mn_major_descriptor(v_addr + k * 2048, L::KV_HALF_BYTES), idesc_o, (t > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(bar(P_EMPTY));            // P may be written again, and O is at rest until the next P is ready
        tcgen05_commit(bar(V_EMPTY, stage));
      }
      if (ok) tcgen05_commit(bar(O_FULL));       // the output is complete
    }
  } else {
    // ------------------------------------------------------------------ softmax, one thread per row
    const int quadrant = warp & 3;
    const int r = quadrant * 32 + lane;                       // row of the tile, lane of tensor memory
    const uint32_t lane_base = tmem_base + ((uint32_t)(quadrant * 32) << 16);
    const int my_pos = pos0 + r;
    float reference = -FLT_MAX, row_sum = 0.f;                // the reference in units of log2, scaled
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t & 1;
      uint8_t* p_row = generic_base + L::P_OFFSET + r * 128;
      const int key0 = kv_begin + t * BKEYS;
      ok = ok && mbar_wait(bar(S_FULL, st), (t >> 1) & 1, abort_flag, p.error, 8);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      // The whole tile is visible to every row of the block: no mask. Otherwise a row sees the
      // keys lo..hi of the request (nothing when the row is past the request's tokens).
      const bool unmasked = key0 + BKEYS - 1 <= pos0 && key0 + BKEYS <= kv_end && key0 >= first_key &&
                            (p.window <= 0 || pos0 + rows - 1 - key0 < p.window);
      const int hi = r < rows ? min(my_pos, kv_end - 1) - key0 : -1;          // relative to the tile
      const int lo = (p.window > 0 ? max(first_key, my_pos - p.window + 1) : first_key) - key0;
      float s[BKEYS];
      tmem_load32(lane_base + st * L::S_COLUMNS, s);
      tmem_load32(lane_base + st * L::S_COLUMNS + 32, s + 32);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(S_EMPTY, st));             // the scores are in registers
      float m4[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};
      if (unmasked) {
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) m4[i & 3] = fmaxf(m4[i & 3], s[i]);
      } else {
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) m4[i & 3] = fmaxf(m4[i & 3], (i >= lo && i <= hi) ? s[i] : -FLT_MAX);
      }
      float tile_max = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      if (tile_max != -FLT_MAX) tile_max *= p.scale_log2;        // the scale is positive: max(s) scales with it
      // The second product of the tile before has completed: P may be written, O is at rest.
      if (t >= 1) ok = mbar_wait(bar(P_EMPTY), (t - 1) & 1, abort_flag, p.error, 7);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const bool moves = tile_max > reference + REFERENCE_SLACK || (reference == -FLT_MAX && tile_max != -FLT_MAX);
      if (__any_sync(0xffffffffu, moves)) {
        // Some row of this warp moves its reference: its sum and its row of O are multiplied
        // by 2^(old - new); the other rows by 1. Reading and writing tensor memory takes the whole warp.
        const float shrink = !moves ? 1.f : (reference == -FLT_MAX ? 0.f : fast_exp2(reference - tile_max));
        if (moves) {
          reference = tile_max;
          row_sum *= shrink;
        }
        if (t >= 1) {
          tcgen05_fence_after();
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            float o[32];
            tmem_load32(lane_base + L::O_COLUMN + c, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= shrink;
            tmem_store32(lane_base + L::O_COLUMN + c, o);
          }
        }
      }
      // exp2(s * scale - reference) as one fused multiply-add and one ex2; a row that has seen
      // no key yet has no reference and every probability 0.
      const float offset = reference == -FLT_MAX ? 0.f : -reference;
      const float factor = reference == -FLT_MAX ? 0.f : p.scale_log2;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      if (unmasked) {
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) {
          s[i] = fast_exp2(fmaf(s[i], factor, offset));
          sum4[i & 3] += s[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < BKEYS; ++i) {
          const float e = fast_exp2(fmaf(s[i], factor, offset));
          s[i] = (i >= lo && i <= hi && factor != 0.f) ? e : 0.f;
          sum4[i & 3] += s[i];
        }
      }
      row_sum += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // 64 keys = eight 16-byte chunks of this row, swizzled by the row.
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 packed;
        __nv_bfloat162* h2 = (__nv_bfloat162*)&packed;
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(s[j * 8 + 2 * e], s[j * 8 + 2 * e + 1]);
        *(uint4*)(p_row + ((j ^ (r & 7)) << 4)) = packed;
      }
      tcgen05_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is for the tensor core's eyes
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_READY));
    }
    ok = __all_sync(0xffffffffu, ok);
    if (active && ok && n_tiles > 0) {
      ok = mbar_wait(bar(O_FULL), 0, abort_flag, p.error, 9);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tcgen05_fence_after();
        const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
        __nv_bfloat16* out = p.out + ((size_t)(first_token + tile * BQ + r) * p.heads + h) * D;
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          float o[32];
          tmem_load32(lane_base + L::O_COLUMN + c, o);        // every lane takes part
          if (r < rows) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 packed;
              __nv_bfloat162* h2 = (__nv_bfloat162*)&packed;
#pragma unroll
              for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(o[j * 8 + 2 * e] * inv, o[j * 8 + 2 * e + 1] * inv);
              *(uint4*)(out + c + j * 8) = packed;
            }
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, L::TMEM_COLUMNS);
  }
}

}  // namespace paired

// ---------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return (EncodeTiled)ptr;
  }();
  return fn;
}

// [rows, cols] bfloat16 row-major as boxes of 64 columns x box_rows rows, 128-byte swizzle.
int tensor_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return fail(101, "paged_attention_tcgen05: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, element_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(102, "paged_attention_tcgen05: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

int sm_count() {
  static int count = [] {
    int device = 0, n = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
    return n;
  }();
  return count;
}

// form 0 picks by the size of the launch: the paired kernel when it has at least two blocks per
// SM; else the wide one, and when its blocks are fewer than half of the SMs (a short portion
// of a prompt over a long context) a query tile's keys are shared out over a cluster of 2, 4 or
// 8 blocks, as long as all blocks still run at once and each has two key tiles or more. A block
// costs about 10 us around its tiles and only one fits an SM, so a second wave of blocks would
// cost more than the shorter chains save: 128 tokens after 8,192 take 123 us in 12 blocks.
// 1: wide, no clusters; 2: paired; 4, 8, 16: wide in clusters of 2, 4, 8.
template <int D>
int launch(const Params& p, const void* qkv, const void* keys, const void* values, int tokens, long long pages, int seqs,
           int working_seqs, int max_q_len, int max_kv_len, int form, int* chosen, cudaStream_t stream) {
  // With a list of the requests to work on, the grid covers those only. Without one it covers
  // all, and the blocks of requests that are left to the decode kernel return at once; they do
  // not count below, but each still costs its launch (one block of 200 KB per SM at a time: 65
  // requests of which one brings a portion took 75 us where that portion needs 15).
  dim3 grid(p.heads, (max_q_len + BQ - 1) / BQ, p.work_index != nullptr ? working_seqs : seqs);
  const long long blocks = (long long)grid.x * grid.y * working_seqs;
  const bool use_paired = form == 2 || (form == 0 && blocks >= 2LL * sm_count());
  unsigned ranks = 1;
  if (form == 4 || form == 8 || form == 16) ranks = form / 2;
  if (form == 0 && !use_paired) {
    const int seen = p.window > 0 && p.window + BQ < max_kv_len ? p.window + BQ : max_kv_len;
    const int longest = (seen + BKEYS - 1) / BKEYS;        // key tiles of the longest block
    while (ranks < 8 && blocks * (ranks * 2) <= sm_count() && longest >= (int)(ranks * 2) * 2) ranks *= 2;
  }
  CUtensorMap map_q, map_k, map_v;
  if (int err = tensor_map(&map_q, qkv, tokens, (p.heads + 2 * p.kv_heads) * D, BQ)) return err;
  const long long cache_rows = pages * p.kv_heads * p.page_size;
  const int tile_keys = use_paired ? paired::BKEYS : BKEYS;
  const int box_rows = p.page_size < tile_keys ? p.page_size : tile_keys;
  if (int err = tensor_map(&map_k, keys, cache_rows, D, box_rows)) return err;
  if (int err = tensor_map(&map_v, values, cache_rows, D, box_rows)) return err;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(prefill_tcgen05_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Layout<D>::SMEM_BYTES);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(prefill_tcgen05_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Layout<D>::SMEM_BYTES);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(paired::prefill_tcgen05_paired_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)paired::Layout<D>::SMEM_BYTES);
    if (err != cudaSuccess) return fail(100, "paged_attention_tcgen05: %s", cudaGetErrorString(err));
    configured = true;
  }
  if (chosen != nullptr) *chosen = use_paired ? 0 : (int)ranks;
  if (use_paired) {
    launch_kernel(paired::prefill_tcgen05_paired_kernel<D>, grid, paired::THREADS, paired::Layout<D>::SMEM_BYTES, stream, map_q, map_k,
                  map_v, p);
  } else {
    grid.x *= ranks;
    if (ranks > 1)
      launch_kernel_cluster(prefill_tcgen05_kernel<D, true>, grid, dim3(THREADS), Layout<D>::SMEM_BYTES, stream, ranks, map_q, map_k, map_v, p);
    else
      launch_kernel(prefill_tcgen05_kernel<D, false>, grid, THREADS, Layout<D>::SMEM_BYTES, stream, map_q, map_k, map_v, p);
  }
  return check_launch("paged_attention_tcgen05");
}

}  // namespace

PAE_EXPORT int pae_attention_tcgen05_supports(int heads, int kv_heads, int d, int page_size) {
  return (d == 64 || d == 128) && (page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128) &&
         kv_heads >= 1 && heads % kv_heads == 0;
}

// Attention of every request that brings more than one token (or every request, unless
// skip_single; `singles` is how many bring one, -1 when the caller does not know). form 0 picks the kernel by the size of the launch, 1 and 2 name it (tests); `chosen` (a host pointer, or null) receives the blocks per query tile of this launch: 1 without clusters, 0 for the paired kernel. `work_index` (device, or null) lists the `work_count` requests that the launch is to cover, in place of all `seqs`. qkv [tokens, heads + 2 kv_heads, d]; keys, values [pages, kv_heads, page_size, d].
PAE_EXPORT int pae_paged_attention_prefill_tcgen05(void* out, const void* qkv, const void* keys, const void* values,
                                                   long long pages, const int* block_table, int table_width,
                                                   const int* q_start, const int* q_pos0, const int* kv_len, int tokens,
                                                   int seqs, int max_q_len, int max_kv_len, int heads, int kv_heads, int d,
                                                   int page_size, float scale, int window, int skip_single, int singles, int form, int* chosen,
                                                   const int* work_index, int work_count, int* error, void* stream) {
  if (seqs == 0 || max_q_len == 0 || tokens == 0) return 0;
  if (work_index != nullptr && (work_count < 1 || work_count > seqs))
    return fail(2, "paged_attention_tcgen05: a list of %d requests to work on, of %d", work_count, seqs);
  if (!pae_attention_tcgen05_supports(heads, kv_heads, d, page_size))
    return fail(2, "paged_attention_tcgen05: head_dim %d with pages of %d is not taken (64 or 128; 16, 32, 64 or 128)", d, page_size);
  if (heads > 65535 || seqs > 65535) return fail(3, "paged_attention_tcgen05: %d heads x %d requests exceed one launch", heads, seqs);
  if ((((uintptr_t)qkv | (uintptr_t)keys | (uintptr_t)values | (uintptr_t)out) & 15) != 0)
    return fail(2, "paged_attention_tcgen05: an operand does not start on a 16-byte boundary");
  Params p{};
  p.out = (__nv_bfloat16*)out;
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
  p.scale_log2 = scale * LOG2E;
  p.error = error;
  cudaStream_t s = (cudaStream_t)stream;
  p.work_index = work_index;
  const int working_seqs = work_index != nullptr ? work_count : (skip_single && singles > 0 && singles < seqs ? seqs - singles : seqs);
  if (d == 64) return launch<64>(p, qkv, keys, values, tokens, pages, seqs, working_seqs, max_q_len, max_kv_len, form, chosen, s);
  return launch<128>(p, qkv, keys, values, tokens, pages, seqs, working_seqs, max_q_len, max_kv_len, form, chosen, s);
}

PAE_DEFINE_LAST_ERROR()

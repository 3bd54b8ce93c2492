// Matrix products of the bfloat16 path on the fifth-generation tensor cores (sm_100a):
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle),
// tcgen05.mma issued by one thread with the accumulator in tensor memory, tcgen05.ld for
// the epilogue. No cluster multicast is used anywhere.
//
// Both operands are K-major ([rows, K] row-major, K contiguous), which is how activations
// [tokens, K] and checkpoint weights [out, K] lie in memory (the reference calls
// F.linear on the same layout, engine/model.py:303-320). One kernel serves two shapes of
// work:
//
//   NORMAL   many tokens (a prompt's portion): the 128 rows of the MMA are tokens, the
//            BN columns are weight rows. out[token, n] = acc (+ bias[n]) (+ residual).
//   SWAPPED  few tokens (decoding): the 128 rows of the MMA are weight rows, the BN >= T
//            columns are the tokens, so a step with 1..64 tokens streams every weight once
//            at full MMA width. K is split over blockIdx.z so that enough blocks are in
//            flight to fill the memory system; each split writes float32 partial sums
//            partial[split, token, n], and the kernel that follows sums them in a fixed
//            order (with bias, residual, or whatever it fuses).
//
// One block computes one 128 x BN tile over its K range. Warp 0 issues the TMA loads,
// warp 1 allocates tensor memory and issues the MMAs, warps 2-5 run the epilogue (each
// reads the 32 lanes of tensor memory that its warp id modulo 4 may touch). Every
// mbarrier wait is bounded: when one gives up it records a code in `error`, the roles
// leave their loops, loads in flight are waited for (bounded again), tensor memory is
// freed and the block returns.
#include "tcgen05.cuh"

using namespace pae;
using namespace pae_tcgen05;

namespace {

constexpr int BM = 128;          // MMA rows per tile
constexpr int THREADS = 192;
constexpr int EPILOGUE_SHARES = 2;           // epilogue warps per quarter of the rows (three were measured slower, one much slower)
constexpr int PERSISTENT_THREADS = 64 + 128 * EPILOGUE_SHARES;     // TMA warp, MMA warp, the epilogue warps
constexpr uint32_t WAIT_LIMIT = 1u << 21;

enum Mode : int { NORMAL = 0, SWAPPED = 1 };

struct Params {
  void* out;
  const float* bias;
  const void* residual;
  int rows_a;        // rows of the A operand (tokens in NORMAL, weight rows in SWAPPED)
  int rows_b;        // rows of the B operand
  int k_blocks;      // ceil(K / 64)
  int kb_per_split;
  int planes;        // persistent kernel: K ranges per output tile, each summed into a float32 plane of its own (0 or 1: none)
  int ld_out;        // NORMAL: row pitch of out/residual in elements; SWAPPED: weight rows N
  int out_f32;
  int swiglu;        // NORMAL only: columns come in blocks of 16 gate, 16 up; out[row, n / 2] = silu(gate) * up
  // q|k|v with rotation and page write in the epilogue (NORMAL, many tokens): out is
  // qkv [tokens, (heads + 2 kv_heads) d]; a tile of 256 columns holds whole heads.
  int rotary;
  const float* rotary_table;   // [tokens, d]: cos of the d/2 frequencies, then sin; or null
  const int* slots;            // [tokens]: page * page_size + offset, negative: no write; or null
  __nv_bfloat16* keys;         // [pages, kv_heads, page_size, d]
  __nv_bfloat16* values;
  int heads, kv_heads, head_dim, page_size;
  int* error;
  int skip_kb;       // self-test of the give-up path only: the k-block (of each block's range) that is never loaded
};

// Waits for a phase of an mbarrier, at most WAIT_LIMIT polls. On giving up it raises the
// block's abort flag and records `code`; it also returns false as soon as another role
// has raised the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error, int code,
                                          uint32_t limit = WAIT_LIMIT) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (i > 64) __nanosleep(64);
  }
  *abort_flag = 1;
  atomicCAS(error, 0, code);
  return false;
}

// One thread's 16 consecutive outputs of row `row` from column `col0` on: bias, residual,
// rounding, store (16-byte stores when the row pitch allows).
__device__ __forceinline__ void store_row_chunk(const Params& p, int row, int col0, float* v, size_t plane_offset = 0) {
    const int valid = min(16, p.rows_b - col0);
    if (p.bias != nullptr) {
      if (valid == 16 && (((uintptr_t)(p.bias + col0)) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 b = *(const float4*)(p.bias + col0 + 4 * q);
          v[4 * q] += b.x; v[4 * q + 1] += b.y; v[4 * q + 2] += b.z; v[4 * q + 3] += b.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < valid) v[i] += p.bias[col0 + i];
      }
    }
    const size_t at = plane_offset + (size_t)row * p.ld_out + col0;
    if (p.out_f32) {
      float* out = (float*)p.out + at;
      if (p.residual != nullptr) {
        const float* res = (const float*)p.residual + at;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < valid) v[i] += res[i];
      }
      if (valid == 16 && (at & 3) == 0) {
#pragma unroll
        for (int i = 0; i < 16; i += 4) *(float4*)(out + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < valid) out[i] = v[i];
      }
    } else {
      __nv_bfloat16* out = (__nv_bfloat16*)p.out + at;
      if (p.residual != nullptr) {
        const __nv_bfloat16* res = (const __nv_bfloat16*)p.residual + at;
        if (valid == 16 && (at & 7) == 0) {
          uint4 r0 = *(const uint4*)res, r1 = *(const uint4*)(res + 8);
          const __nv_bfloat16* rr0 = (const __nv_bfloat16*)&r0;
          const __nv_bfloat16* rr1 = (const __nv_bfloat16*)&r1;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] += __bfloat162float(rr0[i]);
            v[8 + i] += __bfloat162float(rr1[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < valid) v[i] += __bfloat162float(res[i]);
        }
      }
      if (valid == 16 && (at & 7) == 0) {
        uint4 w0, w1;
        __nv_bfloat162* h0 = (__nv_bfloat162*)&w0;
        __nv_bfloat162* h1 = (__nv_bfloat162*)&w1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          h0[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
          h1[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]);
        }
        *(uint4*)out = w0;
        *(uint4*)(out + 8) = w1;
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < valid) out[i] = __float2bfloat16_rn(v[i]);
      }
    }
}

// SwiGLU in the epilogue: 16 gate columns and the 16 up columns that follow them give 16
// outputs. Gate and up are rounded to bfloat16 first, as the unfused path stores them.
__device__ __forceinline__ void store_swiglu_chunk(const Params& p, int row, int col0, const float* g, const float* u) {
  __nv_bfloat16* out = (__nv_bfloat16*)p.out + (size_t)row * p.ld_out + (col0 >> 1);
  uint4 w0, w1;
  __nv_bfloat162* h0 = (__nv_bfloat162*)&w0;
  __nv_bfloat162* h1 = (__nv_bfloat162*)&w1;
  float r[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float gg = __bfloat162float(__float2bfloat16_rn(g[i]));
    const float uu = __bfloat162float(__float2bfloat16_rn(u[i]));
    r[i] = gg / (1.f + expf(-gg)) * uu;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h0[i] = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
    h1[i] = __floats2bfloat162_rn(r[8 + 2 * i], r[8 + 2 * i + 1]);
  }
  *(uint4*)out = w0;
  *(uint4*)(out + 8) = w1;
}


// q|k|v in the epilogue: 16 columns `lo` of a head's first half and the 16 columns `hi` that
// stand d/2 further, of token `row`. Bias, rounding to bfloat16, rotation of q and k
// (engine/model.py:155-161: lo' = lo c - hi s, hi' = hi c + lo s), then qkv and, for k and v,
// the token's place in its page. The same arithmetic as the stand-alone kernels.
// The cosines and sines of 16 frequencies from `f0` on of token `row`.
__device__ __forceinline__ void load_angles(const Params& p, int row, int f0, float* cs, float* sn) {
  const int d = p.head_dim;
  const float4* cos4 = (const float4*)(p.rotary_table + (size_t)row * d + f0);
  const float4* sin4 = (const float4*)(p.rotary_table + (size_t)row * d + (d >> 1) + f0);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 c = cos4[q], sv = sin4[q];
    cs[q * 4] = c.x; cs[q * 4 + 1] = c.y; cs[q * 4 + 2] = c.z; cs[q * 4 + 3] = c.w;
    sn[q * 4] = sv.x; sn[q * 4 + 1] = sv.y; sn[q * 4 + 2] = sv.z; sn[q * 4 + 3] = sv.w;
  }
}

__device__ __forceinline__ void store_rotary_chunks(const Params& p, int row, int head, int f0, float* lo, float* hi,
                                                    const float* cs, const float* sn, int slot) {
  const int d = p.head_dim, half = d >> 1;
  const int col_lo = head * d + f0, col_hi = col_lo + half;
  if (p.bias != nullptr) {
    if (((uintptr_t)(p.bias + col_lo) & 15) == 0 && ((uintptr_t)(p.bias + col_hi) & 15) == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 a = *(const float4*)(p.bias + col_lo + 4 * q), b = *(const float4*)(p.bias + col_hi + 4 * q);
        lo[4 * q] += a.x; lo[4 * q + 1] += a.y; lo[4 * q + 2] += a.z; lo[4 * q + 3] += a.w;
        hi[4 * q] += b.x; hi[4 * q + 1] += b.y; hi[4 * q + 2] += b.z; hi[4 * q + 3] += b.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        lo[i] += p.bias[col_lo + i];
        hi[i] += p.bias[col_hi + i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    lo[i] = __bfloat162float(__float2bfloat16_rn(lo[i]));
    hi[i] = __bfloat162float(__float2bfloat16_rn(hi[i]));
  }
  if (p.rotary_table != nullptr && head < p.heads + p.kv_heads) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      rotate_pair(lo[i], hi[i], cs[i], sn[i]);
    }
  }
  uint4 packed[4];
  __nv_bfloat162* h2 = (__nv_bfloat162*)packed;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    h2[i] = __floats2bfloat162_rn(lo[2 * i], lo[2 * i + 1]);
    h2[8 + i] = __floats2bfloat162_rn(hi[2 * i], hi[2 * i + 1]);
  }
  __nv_bfloat16* out = (__nv_bfloat16*)p.out + (size_t)row * p.ld_out;
  *(uint4*)(out + col_lo) = packed[0];
  *(uint4*)(out + col_lo + 8) = packed[1];
  *(uint4*)(out + col_hi) = packed[2];
  *(uint4*)(out + col_hi + 8) = packed[3];
  if (head >= p.heads) {
    if (slot >= 0 && slot_in_pool(slot, p.page_size)) {
      const int page = slot / p.page_size, offset = slot - page * p.page_size;
      const bool is_key = head < p.heads + p.kv_heads;
      const int kv_head = is_key ? head - p.heads : head - p.heads - p.kv_heads;
      __nv_bfloat16* to = (is_key ? p.keys : p.values) + (((size_t)page * p.kv_heads + kv_head) * p.page_size + offset) * d;
      *(uint4*)(to + f0) = packed[0];
      *(uint4*)(to + f0 + 8) = packed[1];
      *(uint4*)(to + half + f0) = packed[2];
      *(uint4*)(to + half + f0 + 8) = packed[3];
    }
  }
}

template <int BN>
struct Tile {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // As many stages as fit beside a second resident block (about 100 KB each), at most 8.
  static constexpr int STAGES = (100 * 1024 / STAGE_BYTES) > 8 ? 8 : (100 * 1024 / STAGE_BYTES < 2 ? 2 : 100 * 1024 / STAGE_BYTES);
  static constexpr int TMEM_COLUMNS = BN < 32 ? 32 : BN;
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
};

// SELFTEST is the kernel with which a test makes a wait run out, to see the give-up path work:
// the producer never loads k-block `p.skip_kb` (nothing is in flight for it, its barrier is
// never armed), so the MMA issuer's wait for that stage reaches its limit (a short one here),
// raises the abort flag and the error word, and every role leaves through the same code as in
// the product: loads in flight are waited for, tensor memory is freed, the block returns.
constexpr uint32_t SELFTEST_WAIT_LIMIT = 1u << 12;

template <int BN, int MODE, bool SELFTEST = false>
__global__ void __launch_bounds__(THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b, const Params p) {
  using T = Tile<BN>;
  constexpr uint32_t limit = SELFTEST ? SELFTEST_WAIT_LIMIT : WAIT_LIMIT;
  extern __shared__ uint8_t raw_smem[];
  const uint32_t raw = smem_u32(raw_smem);
  const uint32_t base = (raw + 1023u) & ~1023u;                   // swizzled tiles start on 1024 bytes
  uint8_t* generic_base = raw_smem + (base - raw);
  const uint32_t bars = base + T::STAGES * T::STAGE_BYTES;        // full[STAGES], empty[STAGES], tmem_full
  volatile uint32_t* tmem_holder = (volatile uint32_t*)(generic_base + T::STAGES * T::STAGE_BYTES + 8 * (2 * T::STAGES + 1));
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

  dependent_launch_trigger();     // the kernel after this one may begin its own set-up
  if (threadIdx.x == 0) {         // the descriptors do not depend on the kernel before: fetch them early
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x, tile_b = blockIdx.y;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
  const int kb_count = kb_end - kb_begin;

  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (T::STAGES + s); };
  const uint32_t tmem_full_bar = bars + 8u * (2 * T::STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_holder), T::TMEM_COLUMNS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // Barriers and tensor memory are set up. The WEIGHT operand (A when the rows of the MMA are
  // weight rows, else B) is never written during a step, so its first stages are fetched
  // now, while the kernel before this one may still be running; everything else of global
  // memory has to wait for that kernel.
  const int early = min(kb_count, T::STAGES);
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < early; ++i) {
      if (SELFTEST && i == p.skip_kb) continue;
      const uint32_t a_dst = base + i * T::STAGE_BYTES;
      mbar_expect_tx(full_bar(i), T::STAGE_BYTES);
      if (MODE == SWAPPED)
        tma_load_2d(a_dst, &map_a, full_bar(i), (kb_begin + i) * BK, tile_a * BM);
      else
        tma_load_2d(a_dst + T::A_BYTES, &map_b, full_bar(i), (kb_begin + i) * BK, tile_b * BN);
    }
  }
  dependent_launch_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int issued = early;
      for (int i = 0; i < early; ++i) {          // the other operand of the stages begun above
        if (SELFTEST && i == p.skip_kb) continue;
        const uint32_t a_dst = base + i * T::STAGE_BYTES;
        if (MODE == SWAPPED)
          tma_load_2d(a_dst + T::A_BYTES, &map_b, full_bar(i), (kb_begin + i) * BK, tile_b * BN);
        else
          tma_load_2d(a_dst, &map_a, full_bar(i), (kb_begin + i) * BK, tile_a * BM);
      }
      for (int i = early; i < kb_count; ++i) {
        const int s = i % T::STAGES;
        if (!mbar_wait(empty_bar(s), ((i / T::STAGES) - 1) & 1, abort_flag, p.error, 1, limit)) break;
        if (SELFTEST && i == p.skip_kb) continue;
        const uint32_t a_dst = base + s * T::STAGE_BYTES;
        mbar_expect_tx(full_bar(s), T::STAGE_BYTES);
        tma_load_2d(a_dst, &map_a, full_bar(s), (kb_begin + i) * BK, tile_a * BM);
        tma_load_2d(a_dst + T::A_BYTES, &map_b, full_bar(s), (kb_begin + i) * BK, tile_b * BN);
        issued = i + 1;
      }
      if (*abort_flag) {
        // Loads that were issued still write into this block's shared memory: wait for them.
        for (int i = max(0, issued - T::STAGES); i < issued; ++i)
          if (!(SELFTEST && i == p.skip_kb))
          for (uint32_t t = 0; t < WAIT_LIMIT && !mbar_try_wait(full_bar(i % T::STAGES), (i / T::STAGES) & 1); ++t) __nanosleep(64);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instruction_descriptor(BM, BN);
      bool ok = true;
      for (int i = 0; i < kb_count && ok; ++i) {
        const int s = i % T::STAGES;
        ok = mbar_wait(full_bar(s), (i / T::STAGES) & 1, abort_flag, p.error, 2, limit);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a_addr = base + s * T::STAGE_BYTES;
        const uint32_t b_addr = a_addr + T::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // Inside the 128-byte swizzle row a step of 16 elements is 32 bytes.
          umma_bf16(tmem_base, smem_descriptor(a_addr + k * UMMA_K * 2), smem_descriptor(b_addr + k * UMMA_K * 2), idesc,
                    (i > 0 || k > 0) ? 1u : 0u);
        }
        tcgen05_commit(empty_bar(s));      // the stage is free once these MMAs have read it
      }
      if (ok) tcgen05_commit(tmem_full_bar);  // the accumulator is complete once all MMAs are done
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quadrant = warp & 3;                  // the tensor-memory lanes this warp may read
    const int row_in_tile = quadrant * 32 + lane;
    bool ok = true;
    if (kb_count > 0) ok = mbar_wait(tmem_full_bar, 0, abort_flag, p.error, 3, SELFTEST ? 64 * limit : limit);
    ok = __all_sync(0xffffffffu, ok);               // tcgen05.ld below needs the whole warp
    tcgen05_fence_after();
    if (ok) {
      const int row = tile_a * BM + row_in_tile;    // row of the A operand
      const uint32_t lane_address = tmem_base + ((uint32_t)(quadrant * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        if (kb_count > 0) {
          tmem_load16(lane_address + c0, v);        // warp-collective: every lane takes part
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
        const int col0 = tile_b * BN + c0;          // row of the B operand
        if (row >= p.rows_a || col0 >= p.rows_b) continue;
        if (MODE == SWAPPED) {
          // partial[split, token, weight row]: for one token the 32 lanes write 32 neighbours.
          float* out = (float*)p.out + (size_t)blockIdx.z * p.rows_b * p.ld_out;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col0 + i < p.rows_b) out[(size_t)(col0 + i) * p.ld_out + row] = v[i];
        } else {
          store_row_chunk(p, row, col0, v);
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, T::TMEM_COLUMNS);
  }
}

// ---------------------------------------------------------------------------------------
// The many-token product as a persistent kernel: one block per SM walks over 128 x 256
// output tiles. Four 48 KB stages keep about a microsecond of loads in flight; the
// accumulator is double-buffered in tensor memory (2 x 256 columns), so the epilogue of a
// tile (tcgen05.ld, bias, residual, rounding, stores) runs while the MMAs of the next tile
// are issued. Eight warps run it, two for each quarter of the rows: with four the epilogue of
// a tile (SiLU x up above all) took longer than the tile's MMAs and set the pace. Tiles that share a weight tile are neighbours in the walk, so a weight tile
// is read from memory once and found in L2 by the other blocks. When the output has few tiles
// and K is long, a tile's K is shared out over several blocks, each writing a float32 plane.
// ---------------------------------------------------------------------------------------
template <int PBN>
struct PTile {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = PBN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 6 ? 6 : 200 * 1024 / STAGE_BYTES;
  static constexpr int ACC_COLUMNS = 256;       // the two accumulators lie 256 columns apart
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int PBN>
__global__ void __launch_bounds__(PERSISTENT_THREADS) gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                          const __grid_constant__ CUtensorMap map_b,
                                                                          const Params p, int tiles_a, int tiles_b) {
  constexpr int PSTAGES = PTile<PBN>::STAGES;
  constexpr int P_A_BYTES = PTile<PBN>::A_BYTES;
  constexpr int P_STAGE_BYTES = PTile<PBN>::STAGE_BYTES;
  constexpr int ACC = PTile<PBN>::ACC_COLUMNS;
  dependent_launch_trigger();
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  extern __shared__ uint8_t raw_smem[];
  const uint32_t raw = smem_u32(raw_smem);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* generic_base = raw_smem + (base - raw);
  const uint32_t bars = base + PSTAGES * P_STAGE_BYTES;   // full[S], empty[S], tmem_full[2], tmem_empty[2]
  volatile uint32_t* tmem_holder = (volatile uint32_t*)(generic_base + PSTAGES * P_STAGE_BYTES + 8 * (2 * PSTAGES + 4));
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (PSTAGES + s); };
  auto tmem_full_bar = [&](int a) { return bars + 8u * (2 * PSTAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bars + 8u * (2 * PSTAGES + 2 + a); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), PERSISTENT_THREADS - 64);       // every epilogue thread arrives
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_holder), 2 * ACC);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  dependent_launch_wait();

  // A work item is an output tile, or one of the `planes` ranges of K of an output tile when a
  // launch of few tiles and a long K shares each tile out over several blocks.
  const int planes = p.planes > 1 ? p.planes : 1;
  const int total_items = tiles_a * tiles_b * planes;
  const int k_blocks = p.k_blocks;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int tile = item / planes, kb_first = (item % planes) * p.kb_per_split;
        const int kb_end = min(kb_first + p.kb_per_split, k_blocks);
        const int tile_a = tile % tiles_a, tile_b = tile / tiles_a;     // neighbours share the weight tile
        for (int kb = kb_first; kb < kb_end; ++kb, ++it) {
          const int s = it % PSTAGES;
          if (it >= PSTAGES && !mbar_wait(empty_bar(s), ((it / PSTAGES) - 1) & 1, abort_flag, p.error, 1)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = base + s * P_STAGE_BYTES;
          mbar_expect_tx(full_bar(s), P_STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * BK, tile_a * BM);
          tma_load_2d(a_dst + P_A_BYTES, &map_b, full_bar(s), kb * BK, tile_b * PBN);
        }
      }
      if (*abort_flag) {
        for (int i = max(0, it - PSTAGES); i < it; ++i)
          for (uint32_t t = 0; t < WAIT_LIMIT && !mbar_try_wait(full_bar(i % PSTAGES), (i / PSTAGES) & 1); ++t) __nanosleep(64);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instruction_descriptor(BM, PBN);
      // This one thread's instruction stream paces the tensor core (four MMAs of a k-block run
      // about as long as issuing them takes), so it is kept short: the stage index and its
      // phase are counted, not divided out, and the operand descriptors of a stage are the
      // first stage's plus a multiple of the stage size in the address field (bits 0-13, in
      // units of 16 bytes; the stages lie below 256 KB, so nothing carries out of the field).
      const uint64_t a_desc0 = smem_descriptor(base);
      const uint64_t b_desc0 = smem_descriptor(base + P_A_BYTES);
      int local = 0, s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++local) {
        const int acc = local & 1, use = local >> 1;
        if (local >= 2) ok = mbar_wait(tmem_empty_bar(acc), (use - 1) & 1, abort_flag, p.error, 4);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * ACC;
        const int kb_first = (item % planes) * p.kb_per_split;
        const int kb_count = min(kb_first + p.kb_per_split, k_blocks) - kb_first;
        for (int kb = 0; kb < kb_count; ++kb) {
          if (!mbar_try_wait(full_bar(s), phase)) ok = mbar_wait(full_bar(s), phase, abort_flag, p.error, 2);
          if (!ok) break;
          tcgen05_fence_after();
          const uint64_t stage_offset = (uint64_t)(uint32_t)(s * (P_STAGE_BYTES >> 4));
          const uint64_t a_desc = a_desc0 + stage_offset, b_desc = b_desc0 + stage_offset;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_acc, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit(empty_bar(s));
          if (++s == PSTAGES) {
            s = 0;
            phase ^= 1u;
          }
        }
        if (ok) tcgen05_commit(tmem_full_bar(acc));
      }
    }
  } else {
    const int quadrant = warp & 3;
    const int share = (warp - 2) >> 2;              // which of the warps of this quarter
    const int row_in_tile = quadrant * 32 + lane;
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++local) {
      const int tile = item / planes;
      const size_t plane_offset = (size_t)(item % planes) * p.rows_a * p.ld_out;
      const int tile_a = tile % tiles_a, tile_b = tile / tiles_a;
      const int acc = local & 1, use = local >> 1;
      const int row = tile_a * BM + row_in_tile;
      // What the rotation needs of this thread's token is asked for before the wait for the
      // tile's MMAs: its place in its page and its first 16 cosines and sines.
      const bool rotating = p.rotary && p.rotary_table != nullptr && row < p.rows_a;
      float cs_a[16], sn_a[16];
      int slot = -1;
      if (rotating) load_angles(p, row, 0, cs_a, sn_a);
      if (p.rotary && p.slots != nullptr && row < p.rows_a) slot = p.slots[row];
      ok = ok && mbar_wait(tmem_full_bar(acc), use & 1, abort_flag, p.error, 3);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t lane_address = tmem_base + ((uint32_t)(quadrant * 32) << 16) + acc * ACC;
      // The warps of a quarter of the rows share the tile's columns in equal ranges that end
      // on a multiple of 32 columns (a gate block with its up block) or of the head size.
      const int unit = p.rotary ? p.head_dim : 32;
      const int range = ((PBN + EPILOGUE_SHARES - 1) / EPILOGUE_SHARES + unit - 1) / unit * unit;
      const int col_begin = min(share * range, PBN), col_end = min(col_begin + range, PBN);
      if (p.rotary) {
        // 16 columns of each half of a head at a time; the token's cosines and sines of those
        // 16 frequencies are read once and serve every head of the tile, and those of the next
        // 16 are on their way while these are used.
        const int d = p.head_dim, half = d >> 1;
        auto heads_of = [&](int f0, const float* cs, const float* sn) {
#pragma unroll 1
          for (int head0 = col_begin; head0 < col_end; head0 += d) {
            float lo[16], hi[16];
            tmem_load16(lane_address + head0 + f0, lo);
            tmem_load16(lane_address + head0 + half + f0, hi);
            if (row < p.rows_a && tile_b * PBN + head0 < p.rows_b)
              store_rotary_chunks(p, row, (tile_b * PBN + head0) / d, f0, lo, hi, cs, sn, slot);
          }
        };
#pragma unroll 1
        for (int f0 = 0; f0 < half; f0 += 32) {
          float cs_b[16], sn_b[16];
          const bool second = f0 + 16 < half;
          if (second && rotating) load_angles(p, row, f0 + 16, cs_b, sn_b);
          heads_of(f0, cs_a, sn_a);
          if (second) {
            if (f0 + 32 < half && rotating) load_angles(p, row, f0 + 32, cs_a, sn_a);
            heads_of(f0 + 16, cs_b, sn_b);
          }
        }
      } else if (p.swiglu) {
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end; c0 += 32) {
          float gate[16], up[16];
          tmem_load16(lane_address + c0, gate);
          tmem_load16(lane_address + c0 + 16, up);
          const int col0 = tile_b * PBN + c0;
          if (row < p.rows_a && col0 < p.rows_b) store_swiglu_chunk(p, row, col0, gate, up);
        }
      } else {
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end; c0 += 16) {
          float v[16];
          tmem_load16(lane_address + c0, v);
          const int col0 = tile_b * PBN + c0;
          if (row < p.rows_a && col0 < p.rows_b) store_row_chunk(p, row, col0, v, plane_offset);
        }
      }
      tcgen05_fence_before();
      mbar_arrive(tmem_empty_bar(acc));        // this thread has read its part of the accumulator
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 2 * ACC);
  }
}

// ---------------------------------------------------------------------------------------
// Host side: tensor maps (cached by pointer and shape), launch.
// ---------------------------------------------------------------------------------------
template <int BN, int MODE, bool SELFTEST = false>
int launch(const Params& p, const void* a, const void* b, int k, int splits, cudaStream_t stream) {
  using T = Tile<BN>;
  CUtensorMap map_a, map_b;
  if (int err = tensor_map(&map_a, a, p.rows_a, k, BM)) return err;
  if (int err = tensor_map(&map_b, b, p.rows_b, k, BN)) return err;
  auto kernel = gemm_tcgen05_kernel<BN, MODE, SELFTEST>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM_BYTES);
    if (err != cudaSuccess) return fail(100, "linear_tcgen05: %s", cudaGetErrorString(err));
    configured = true;
  }
  dim3 grid((p.rows_a + BM - 1) / BM, (p.rows_b + BN - 1) / BN, splits);
  launch_kernel(kernel, grid, THREADS, T::SMEM_BYTES, stream, map_a, map_b, p);
  return check_launch("linear_tcgen05");
}

int sm_count() {
  static int count = [] {
    int device = 0, n = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
    return n;
  }();
  return count;
}

template <int PBN>
int launch_persistent_with(const Params& p, const void* a, const void* b, int k, cudaStream_t stream) {
  using T = PTile<PBN>;
  CUtensorMap map_a, map_b;
  if (int err = tensor_map(&map_a, a, p.rows_a, k, BM)) return err;
  if (int err = tensor_map(&map_b, b, p.rows_b, k, PBN)) return err;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<PBN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM_BYTES);
    if (err != cudaSuccess) return fail(100, "linear_tcgen05: %s", cudaGetErrorString(err));
    configured = true;
  }
  const int tiles_a = (p.rows_a + BM - 1) / BM, tiles_b = (p.rows_b + PBN - 1) / PBN;
  const int items = tiles_a * tiles_b * (p.planes > 1 ? p.planes : 1);
  const int blocks = items < sm_count() ? items : sm_count();
  launch_kernel(gemm_tcgen05_persistent_kernel<PBN>, dim3(blocks), PERSISTENT_THREADS, T::SMEM_BYTES, stream, map_a, map_b, p, tiles_a, tiles_b);
  return check_launch("linear_tcgen05");
}

// The tile width whose walk over the output costs least: rounds of tiles over the SMs
// times (width + a fixed share for a tile's first loads and its epilogue). The narrow widths
// serve a portion of a few hundred tokens, whose few wide tiles would leave most SMs idle
// (q|k|v of 128 tokens: 8 tiles of 256 columns, 18.1 us with 16 of 128 against 23.7); they are
// left out where a long K is shared out over blocks instead (a plain product with 32 k-blocks
// and more: `pae_linear_tcgen05_plane_count`), because a narrow tile reads the tokens' operand
// from L2 once more per 64 columns (down of 512 tokens: 42 us with 96 tiles of 64 columns and
// the whole K each, 21.5 us with 36 tiles of 176 in four planes).
int persistent_width(const Params& p) {
  const int widths[5] = {256, 192, 176, 128, 64};
  const int tiles_a = (p.rows_a + BM - 1) / BM;
  const bool narrow = p.swiglu || p.rotary || p.k_blocks < 32;
  int best = 256;
  long best_cost = -1;
  for (int w : widths) {
    if (w < 176 && !narrow) continue;
    if (p.swiglu && w % 32) continue;         // a tile must not cut a gate block from its up block
    if (p.rotary && w % p.head_dim) continue; // nor a head
    const int tiles = tiles_a * ((p.rows_b + w - 1) / w);
    const long cost = (long)((tiles + sm_count() - 1) / sm_count()) * (w + 32);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = w;
    }
  }
  return best;
}

int launch_persistent(const Params& p, const void* a, const void* b, int k, cudaStream_t stream) {
  const int best = persistent_width(p);
  if (best == 192) return launch_persistent_with<192>(p, a, b, k, stream);
  if (best == 176) return launch_persistent_with<176>(p, a, b, k, stream);
  if (best == 128) return launch_persistent_with<128>(p, a, b, k, stream);
  if (best == 64) return launch_persistent_with<64>(p, a, b, k, stream);
  return launch_persistent_with<256>(p, a, b, k, stream);
}

int check_operands(const void* x, const void* w, int k) {
  if (k % 8) return fail(2, "linear_tcgen05: K = %d is not a multiple of 8 (a TMA row pitch must be a multiple of 16 bytes)", k);
  if (((uintptr_t)x | (uintptr_t)w) & 15) return fail(2, "linear_tcgen05: an operand does not start on a 16-byte boundary");
  return 0;
}

}  // namespace

// out[tokens, n] = x[tokens, k] . w[n, k]^T (+ bias[n]) (+ residual[tokens, n]); x, w, residual
// bfloat16, bias float32, out bfloat16 or float32 (then residual is float32 too).
// out[tokens, n / 2] = silu(gate) * up where x . w^T gives gate and up in alternating blocks of 16
// columns (w's rows are laid out that way); many tokens only (the persistent kernel). n is a
// multiple of 32 and at least 256.
PAE_EXPORT int pae_linear_swiglu_tcgen05(void* out, const void* x, const void* w, int tokens, int n, int k, int* error,
                                         void* stream) {
  if (tokens == 0 || n == 0) return 0;
  if (n % 32 || n < 256) return fail(2, "linear_swiglu_tcgen05: %d columns are not a multiple of 32 of at least 256", n);
  if (int err = check_operands(x, w, k)) return err;
  Params p{};
  p.out = out;
  p.rows_a = tokens;
  p.rows_b = n;
  p.k_blocks = (k + BK - 1) / BK;
  p.kb_per_split = p.k_blocks;
  p.ld_out = n / 2;
  p.swiglu = 1;
  p.error = error;
  return launch_persistent(p, x, w, k, (cudaStream_t)stream);
}

// 1 when the many-token product can finish q|k|v itself for this head size.
PAE_EXPORT int pae_linear_rotary_tcgen05_supports(int d) { return d >= 32 && d % 32 == 0 && 256 % d == 0; }

// qkv[tokens, n] = x . w^T + bias with n = (heads + 2 kv_heads) d, q and k rotated by
// rotary [tokens, d] (or not, when null), and k and v also written to their pages at `slots`
// (or not, when null): the product, `pae_rotary_qk_cache_write` and the page write in one
// kernel. Many tokens only (more than 64); head sizes that divide 256.
PAE_EXPORT int pae_linear_rotary_tcgen05(void* qkv, const void* x, const void* w, const float* bias, const float* rotary,
                                         const int* slots, void* keys, void* values, int tokens, int heads, int kv_heads,
                                         int d, int page_size, int k, int* error, void* stream) {
  const int n = (heads + 2 * kv_heads) * d;
  if (tokens == 0 || n == 0) return 0;
  if (!pae_linear_rotary_tcgen05_supports(d)) return fail(2, "linear_rotary_tcgen05: head_dim %d does not divide 256 in steps of 32", d);
  if (n < 256) return fail(2, "linear_rotary_tcgen05: %d columns are fewer than the 256 of a tile", n);
  if (slots != nullptr && (keys == nullptr || values == nullptr || page_size < 1))
    return fail(2, "linear_rotary_tcgen05: slots without pages");
  if (((uintptr_t)qkv | (uintptr_t)keys | (uintptr_t)values | (uintptr_t)rotary) & 15)
    return fail(2, "linear_rotary_tcgen05: an operand does not start on a 16-byte boundary");
  if (int err = check_operands(x, w, k)) return err;
  Params p{};
  p.out = qkv;
  p.bias = bias;
  p.rows_a = tokens;
  p.rows_b = n;
  p.k_blocks = (k + BK - 1) / BK;
  p.kb_per_split = p.k_blocks;
  p.ld_out = n;
  p.rotary = 1;
  p.rotary_table = rotary;
  p.slots = slots;
  p.keys = (__nv_bfloat16*)keys;
  p.values = (__nv_bfloat16*)values;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.head_dim = d;
  p.page_size = page_size;
  p.error = error;
  return launch_persistent(p, x, w, k, (cudaStream_t)stream);
}

PAE_EXPORT int pae_linear_tcgen05(void* out, const void* x, const void* w, const float* bias, const void* residual,
                                  int tokens, int n, int k, int out_f32, int* error, void* stream) {
  if (tokens == 0 || n == 0) return 0;
  if (int err = check_operands(x, w, k)) return err;
  Params p{};
  p.out = out;
  p.bias = bias;
  p.residual = residual;
  p.rows_a = tokens;
  p.rows_b = n;
  p.k_blocks = (k + BK - 1) / BK;
  p.kb_per_split = p.k_blocks;
  p.ld_out = n;
  p.out_f32 = out_f32;
  p.error = error;
  cudaStream_t s = (cudaStream_t)stream;
  if (n >= 256) return launch_persistent(p, x, w, k, s);
  if (n >= 128) return launch<128, NORMAL>(p, x, w, k, 1, s);
  if (n > 32) return launch<64, NORMAL>(p, x, w, k, 1, s);
  return launch<32, NORMAL>(p, x, w, k, 1, s);
}

// How many float32 planes `pae_linear_tcgen05_planes` writes for this shape: 1 (call
// `pae_linear_tcgen05` instead) unless the output has so few tiles that they leave more than
// half of the SMs idle (a projection for one or two hundred tokens; a down projection for a few
// hundred): then each tile's K is shared out over as many blocks as fill the SMs, 8 k-blocks
// each at least where K is long (32 k-blocks and more), 4 where it is short. What a block can
// draw from memory is a fraction of what the GPU can, so a product of few tiles runs at the
// speed of few SMs whatever its size (q|k|v of 128 tokens on 16 tiles: 18 us for 6 MB of weights).
PAE_EXPORT int pae_linear_tcgen05_plane_count(int tokens, int n, int k) {
  const int k_blocks = (k + BK - 1) / BK;
  if (tokens <= 64 || n < 256 || k_blocks < 8) return 1;
  const int least = k_blocks >= 32 ? 8 : 4;
  Params p{};
  p.rows_a = tokens;
  p.rows_b = n;
  p.k_blocks = k_blocks;
  const int width = persistent_width(p);
  const int tiles = ((tokens + BM - 1) / BM) * ((n + width - 1) / width);
  if (tiles * 2 > sm_count()) return 1;
  int planes = sm_count() / tiles;
  planes = planes > k_blocks / least ? k_blocks / least : planes;
  if (planes < 2) return 1;
  const int per = (k_blocks + planes - 1) / planes;
  return (k_blocks + per - 1) / per;
}

// partial[plane, token, n] (float32) = x[tokens, k_range(plane)] . w[n, k_range(plane)]^T with
// planes = pae_linear_tcgen05_plane_count(tokens, n, k) > 1; the caller adds the planes up.
PAE_EXPORT int pae_linear_tcgen05_planes(float* partial, const void* x, const void* w, int tokens, int n, int k, int planes,
                                         int* error, void* stream) {
  if (tokens == 0 || n == 0) return 0;
  if (int err = check_operands(x, w, k)) return err;
  if (planes < 2 || planes != pae_linear_tcgen05_plane_count(tokens, n, k))
    return fail(2, "linear_tcgen05_planes: %d planes for [%d, %d] x [%d, %d]", planes, tokens, k, n, k);
  Params p{};
  p.out = partial;
  p.rows_a = tokens;
  p.rows_b = n;
  p.k_blocks = (k + BK - 1) / BK;
  p.kb_per_split = (p.k_blocks + planes - 1) / planes;
  p.planes = planes;
  p.ld_out = n;
  p.out_f32 = 1;
  p.error = error;
  return launch_persistent(p, x, w, k, (cudaStream_t)stream);
}

// How many float32 partial planes `pae_linear_tcgen05_swapped` writes for this shape.
PAE_EXPORT int pae_linear_swapped_splits(int n, int k) {
  // Two blocks of this form fit on each SM. The work should fill that one wave
  // (a second, partly filled wave costs a whole block's latency), with at least two k-blocks
  // per split. The count depends on the weight's shape alone, never on the tokens.
  const int tiles = (n + BM - 1) / BM;
  const int k_blocks = (k + BK - 1) / BK;
  int splits = (2 * sm_count()) / tiles;
  splits = splits < 1 ? 1 : splits;
  const int most = k_blocks / 2 < 1 ? 1 : k_blocks / 2;
  splits = splits > most ? most : splits;
  const int per = (k_blocks + splits - 1) / splits;
  return (k_blocks + per - 1) / per;
}

// partial[split, token, n] (float32) = x[tokens, k_split] . w[n, k_split]^T for tokens <= 64.
PAE_EXPORT int pae_linear_tcgen05_swapped(float* partial, const void* x, const void* w, int tokens, int n, int k,
                                          int* error, void* stream) {
  if (tokens == 0 || n == 0) return 0;
  if (tokens > 128) return fail(2, "linear_tcgen05_swapped: %d tokens are more than the 128 it takes", tokens);
  if (int err = check_operands(x, w, k)) return err;
  const int splits = pae_linear_swapped_splits(n, k);
  Params p{};
  p.out = partial;
  p.rows_a = n;
  p.rows_b = tokens;
  p.k_blocks = (k + BK - 1) / BK;
  p.kb_per_split = (p.k_blocks + splits - 1) / splits;
  p.ld_out = n;
  p.out_f32 = 1;
  p.error = error;
  cudaStream_t s = (cudaStream_t)stream;
  if (tokens <= 16) return launch<16, SWAPPED>(p, w, x, k, splits, s);
  if (tokens <= 32) return launch<32, SWAPPED>(p, w, x, k, splits, s);
  if (tokens <= 64) return launch<64, SWAPPED>(p, w, x, k, splits, s);
  return launch<128, SWAPPED>(p, w, x, k, splits, s);
}

// The self-test of the give-up path: `pae_linear_tcgen05_swapped` for at most 16 tokens, except
// that no block ever loads k-block `skip_kb` of its range. Every block's MMA issuer gives up after
// a short wait, the error word gets its role code (2), `partial` holds nothing of use, and the
// kernel returns by itself. Not called by the engine.
PAE_EXPORT int pae_linear_tcgen05_selftest_giveup(float* partial, const void* x, const void* w, int tokens, int n, int k,
                                                   int skip_kb, int* error, void* stream) {
  if (tokens < 1 || tokens > 16 || n < 1) return fail(2, "linear_tcgen05_selftest_giveup: %d tokens (1 to 16), %d rows", tokens, n);
  if (int err = check_operands(x, w, k)) return err;
  const int splits = pae_linear_swapped_splits(n, k);
  Params p{};
  p.out = partial;
  p.rows_a = n;
  p.rows_b = tokens;
  p.k_blocks = (k + BK - 1) / BK;
  p.kb_per_split = (p.k_blocks + splits - 1) / splits;
  if (skip_kb < 0 || skip_kb >= p.kb_per_split) return fail(2, "linear_tcgen05_selftest_giveup: k-block %d of %d", skip_kb, p.kb_per_split);
  p.ld_out = n;
  p.out_f32 = 1;
  p.error = error;
  p.skip_kb = skip_kb;
  return launch<16, SWAPPED, true>(p, w, x, k, splits, (cudaStream_t)stream);
}

PAE_EXPORT int pae_sm_count(void) { return sm_count(); }

// out[token, n] = sum over splits of partial[split, token, n] (+ bias[n]) (+ residual[token, n]),
// summed in the order of the splits. out and residual bfloat16 or float32.
template <typename TO>
__global__ void reduce_splits_kernel(TO* __restrict__ out, const float* __restrict__ partial, const float* __restrict__ bias,
                                     const TO* __restrict__ residual, int splits, long long plane, int n) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= plane) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[(size_t)s * plane + i];
  if (bias != nullptr) v += bias[i % n];
  if (residual != nullptr) v += to_float(residual[i]);
  out[i] = from_float<TO>(v);
}

PAE_EXPORT int pae_reduce_splits(void* out, const float* partial, const float* bias, const void* residual, int splits,
                                 int tokens, int n, int out_f32, void* stream) {
  const long long plane = (long long)tokens * n;
  if (plane == 0) return 0;
  const unsigned blocks = (unsigned)((plane + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_f32)
    launch_kernel(reduce_splits_kernel<float>, blocks, 256, 0, s, (float*)out, partial, bias, (const float*)residual, splits, plane, n);
  else
    launch_kernel(reduce_splits_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, partial, bias, (const __nv_bfloat16*)residual, splits, plane, n);
  return check_launch("reduce_splits");
}

PAE_DEFINE_LAST_ERROR()

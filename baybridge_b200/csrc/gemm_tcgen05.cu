// gemm_tcgen05.cu — BF16 GEMM for sm_100a: C[m,n] = sum_k A'[m,k] * B'[k,n], fp32 accumulate.
//
// Native forms: A is [M,K] (K contiguous) or [K,M] (M contiguous); B is [N,K] (K contiguous, "A · B^T")
// or [K,N] (N contiguous, "A · B") — tcgen05 consumes all four through its K-major / MN-major
// shared-memory descriptors.  Only A stored [K,M] with M not a multiple of 8 (rows that are not 16-byte
// multiples, which TMA cannot read) is brought to [M,K] by a tiled transpose into a workspace.
//
// Kernel structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: streams 128x64 A tiles and 256x64 B tiles (128-byte swizzle) into a
//               4-stage shared-memory ring, signalling `full[stage]` by transaction bytes.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M128 x N256 x K16, both operands
//               from shared memory) into one of two 256-column TMEM accumulators; tcgen05.commit
//               releases ring stages (`empty[stage]`) and publishes finished tiles (`acc_full`).
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator (each warp owns its 32-lane TMEM
//               quadrant), convert, store C; `acc_empty` hands the accumulator back so the next
//               tile's main loop overlaps this tile's epilogue.
// Tensor-core bound: 2*M*N*K flops; per k-block a CTA moves 48 KB of operands for 4.2 MFLOP, so
// operand traffic is served from L2 (tiles are rasterised in groups of 8 M-blocks) and HBM sees
// each operand only a few times.
#include <cuda_bf16.h>

#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "bb200_internal.h"
#include "bb200_sm100.cuh"

namespace bb200 {
namespace {

using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;  // 16 KB
constexpr int ACC_COLUMNS = BN;            // fp32 accumulator of a full-width tile: 128 lanes x 256 columns
constexpr int TMEM_COLUMNS = 2 * ACC_COLUMNS;
constexpr int THREADS = 192;
constexpr int DEFAULT_GROUP_M = 16;        // rasterisation: tiles advance down this many M-blocks before moving in N

// The single-CTA kernel comes in three tile widths.  256 columns is the fastest per flop (one MMA instruction covers
// 128x256); 128 and 64 columns exist for problems with too few 128x256 tiles to occupy the SMs — narrower tiles
// spread the operand streams over more SMs, and their smaller stages buy a deeper ring.
template <int TN> struct Tile {
  static_assert(TN == 256 || TN == 128 || TN == 64, "tile widths: 256, 128, 64");
  static constexpr int STAGES = TN == 256 ? 4 : TN == 128 ? 6 : 8;
  static constexpr int B_TILE_BYTES = TN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int ACC_COLUMNS = TN;          // fp32 accumulator: 128 lanes x TN columns
  static constexpr int TMEM_COLUMNS = 2 * TN;     // double-buffered; a power of two >= 32
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + 4 * 32 * 144 /* epilogue staging */;
};

enum WaitCode { kWaitEmpty = 101, kWaitFull = 102, kWaitAccEmpty = 103, kWaitAccFull = 104 };

// Where the epilogue writes C.  Ordinarily one buffer holding the [m, n] result.  In the gather form the
// [m, n] result of this GPU is one row block of a taller matrix that every GPU of the box holds a copy of:
// the epilogue stores each tile into all `count` copies (its own and, through peer-mapped pointers, the
// others') at row `row_offset`, so the output all-gather rides along with the GEMM tile by tile.
constexpr int kMaxDestinations = 8;
struct Destinations {
  void* p[kMaxDestinations];
  int count;
  int row_offset;
};

struct TileCoord { int m_block, n_block; };

__device__ __forceinline__ TileCoord tile_coord(int tile, int m_blocks, int n_blocks, int group_m) {
  const int group_size = group_m * n_blocks;
  const int group = tile / group_size;
  const int first_m = group * group_m;
  const int rows = min(group_m, m_blocks - first_m);
  const int within = tile - group * group_size;
  return {first_m + within % rows, within / rows};
}

template <typename OutT> __device__ __forceinline__ void store_chunk(OutT* row_ptr, const uint32_t (&acc)[32], int valid);

template <> __device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* row_ptr, const uint32_t (&acc)[32], int valid) {
  if (valid >= 32 && (reinterpret_cast<uintptr_t>(row_ptr) & 15u) == 0) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(acc[v * 8 + 2 * j]), __uint_as_float(acc[v * 8 + 2 * j + 1]));
        packed[j] = *reinterpret_cast<uint32_t*>(&pair);
      }
      *reinterpret_cast<uint4*>(row_ptr + v * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) row_ptr[j] = __float2bfloat16_rn(__uint_as_float(acc[j]));
  }
}

template <> __device__ __forceinline__ void store_chunk<float>(float* row_ptr, const uint32_t (&acc)[32], int valid) {
  if (valid >= 32 && (reinterpret_cast<uintptr_t>(row_ptr) & 15u) == 0) {
#pragma unroll
    for (int v = 0; v < 8; ++v)
      *reinterpret_cast<uint4*>(row_ptr + v * 4) = make_uint4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) row_ptr[j] = __uint_as_float(acc[j]);
  }
}

// ---- epilogue: one warp's 32 accumulator rows x BN columns to every destination ------------------------
// tcgen05.ld 32x32b hands each lane one row, so storing straight from registers would make every warp
// store touch 32 rows with 16 bytes each — tolerable in local HBM (L2 merges sectors), wasteful over NVLink.
// The rows go through a small shared-memory staging area instead (128 bytes per row and pass, rows 144
// bytes apart so neither side has bank conflicts) and leave as 128-byte contiguous row segments: eight lanes
// per row, four rows per store instruction.
constexpr int STAGE_ROW_BYTES = 144;
constexpr int STAGING_BYTES_PER_WARP = 32 * STAGE_ROW_BYTES;
constexpr int STAGING_BYTES = 4 * STAGING_BYTES_PER_WARP;

template <typename OutT, int COLS>
__device__ __forceinline__ void store_accumulator_rows(const Destinations& dst, uint32_t taddr, int first_row, int lane, int m, int n,
                                                       int col0, uint8_t* stage, int extra_row_offset = 0) {
  constexpr int PASS_COLS = 128 / (int)sizeof(OutT);  // columns that make 128 bytes of output: 64 (bf16) or 32 (f32)
  const bool rows_aligned = ((size_t)n * sizeof(OutT)) % 16 == 0;
#pragma unroll 1
  for (int pass = 0; pass < COLS / PASS_COLS; ++pass) {
    uint32_t acc[PASS_COLS];
#pragma unroll
    for (int q = 0; q < PASS_COLS / 32; ++q)
      tmem_ld_32x32b_x32(taddr + (uint32_t)(pass * PASS_COLS + q * 32), *reinterpret_cast<uint32_t(*)[32]>(&acc[q * 32]));
    tmem_ld_wait();
    const int col = col0 + pass * PASS_COLS;
    if (col >= n) continue;
    bool fast = rows_aligned && col + PASS_COLS <= n;
    for (int d = 0; fast && d < dst.count; ++d) fast = (reinterpret_cast<uintptr_t>(dst.p[d]) & 15u) == 0;
    if (fast) {
      uint4* mine = reinterpret_cast<uint4*>(stage + lane * STAGE_ROW_BYTES);
      if constexpr (sizeof(OutT) == 2) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          uint32_t packed[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(acc[v * 8 + 2 * j]), __uint_as_float(acc[v * 8 + 2 * j + 1]));
            packed[j] = *reinterpret_cast<uint32_t*>(&pair);
          }
          mine[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      } else {
#pragma unroll
        for (int v = 0; v < 8; ++v) mine[v] = make_uint4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
      }
      __syncwarp();
      const int piece = lane & 7;  // which 16 bytes of the row's 128
#pragma unroll
      for (int step = 0; step < 8; ++step) {
        const int r = step * 4 + (lane >> 3);
        const uint4 value = *reinterpret_cast<const uint4*>(stage + r * STAGE_ROW_BYTES + piece * 16);
        const int row = first_row + r;
        if (row < m) {
          const size_t byte_offset = ((size_t)(row + dst.row_offset + extra_row_offset) * n + col) * sizeof(OutT) + (size_t)piece * 16;
          for (int d = 0; d < dst.count; ++d) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst.p[d]) + byte_offset) = value;
        }
      }
      __syncwarp();  // the staging rows are rewritten by the next pass
    } else {
      const int row = first_row + lane;
      if (row < m) {
#pragma unroll
        for (int q = 0; q < PASS_COLS / 32; ++q) {
          const int c = col + q * 32;
          if (c < n) {
            const size_t offset = (size_t)(row + dst.row_offset + extra_row_offset) * n + c;
            for (int d = 0; d < dst.count; ++d)
              store_chunk<OutT>(static_cast<OutT*>(dst.p[d]) + offset, *reinterpret_cast<const uint32_t(*)[32]>(&acc[q * 32]), n - c);
          }
        }
      }
    }
  }
}

// B_MN = false: B tile is [BN n-rows, 64 k] (K-major).  B_MN = true: B is stored [K, N]; a stage holds
// BN/64 sub-tiles of [64 k-rows, 64 n] (MN-major), each 8 KB, consecutive in shared memory.  A_MN is the
// same for A stored [K, M]: BM/64 sub-tiles of [64 k-rows, 64 m].
template <typename OutT, bool A_MN, bool B_MN, int TN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_abt_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ Destinations dst,
                int m, int n, int k, int group_m, int splits, int kb_per_split, int* status_word) {
  using T = Tile<TN>;
  constexpr int STAGES = T::STAGES, STAGE_BYTES = T::STAGE_BYTES, ACC_COLUMNS = T::ACC_COLUMNS, TMEM_COLUMNS = T::TMEM_COLUMNS;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern
  const uint32_t smem_base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_addr(smem_raw));
  uint64_t* barriers = reinterpret_cast<uint64_t*>(smem_aligned + STAGES * STAGE_BYTES);
  // barrier layout: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], then the TMEM slot and abort flag
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(barriers + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (m + BM - 1) / BM, n_blocks = (n + TN - 1) / TN;
  const int tiles = m_blocks * n_blocks;
  const int k_blocks = (k + BK - 1) / BK;
  // split along K: work item w covers k-blocks [split * kb_per_split, +kb_per_split) of tile w % tiles and its
  // accumulator goes to row block `split` of an fp32 workspace [splits * m, n] that a second kernel folds
  // (splits == 1: kb_per_split == k_blocks and the tile goes straight to C)
  const int work_items = tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(smem_addr(tmem_slot), TMEM_COLUMNS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; ok && work < work_items; work += gridDim.x) {
        const TileCoord coord = tile_coord(work % tiles, m_blocks, n_blocks, group_m);
        const int kb_begin = (work / tiles) * kb_per_split, kb_end = min(k_blocks, kb_begin + kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          // a fresh barrier's "previous phase" counts as complete: waiting on parity^1 passes at once
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status_word, kWaitEmpty))) break;
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_TILE_BYTES;
          mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
          if constexpr (A_MN) {
#pragma unroll
            for (int t = 0; t < BM / 64; ++t)
              tma_load_2d(a_dst + t * (BK * 128), &map_a, full_bar(stage), coord.m_block * BM + t * 64, kb * BK);
          } else {
            tma_load_2d(a_dst, &map_a, full_bar(stage), kb * BK, coord.m_block * BM);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int t = 0; t < TN / 64; ++t)
              tma_load_2d(b_dst + t * (BK * 128), &map_b, full_bar(stage), coord.n_block * TN + t * 64, kb * BK);
          } else {
            tma_load_2d(b_dst, &map_b, full_bar(stage), kb * BK, coord.n_block * TN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, TN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int work = blockIdx.x; ok && work < work_items; work += gridDim.x, ++local_tile) {
        const int buffer = local_tile & 1;
        const uint32_t acc_phase = (uint32_t)(local_tile >> 1) & 1u;
        if (!(ok = mbar_wait(acc_empty_bar(buffer), acc_phase ^ 1u, abort_flag, status_word, kWaitAccEmpty))) break;
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buffer * ACC_COLUMNS);
        const int kb_begin = (work / tiles) * kb_per_split, kb_end = min(k_blocks, kb_begin + kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, status_word, kWaitFull))) break;
          tcgen05_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE_BYTES;
          const uint64_t desc_a = A_MN ? umma_desc_mn_major_sw128(a_src, BK * 128) : umma_desc_k_major_sw128(a_src);
          const uint64_t desc_b = B_MN ? umma_desc_mn_major_sw128(a_src + A_TILE_BYTES, BK * 128)
                                       : umma_desc_k_major_sw128(a_src + A_TILE_BYTES);
          // one K step of 16: 32 bytes along a K-major row, or 16 rows of 128 bytes in an MN-major tile
          constexpr uint32_t a_step = A_MN ? UMMA_K * 128 : UMMA_K * 2;
          constexpr uint32_t b_step = B_MN ? UMMA_K * 128 : UMMA_K * 2;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_bf16_ss(tmem_acc, umma_desc_advance_k(desc_a, kk * a_step), umma_desc_advance_k(desc_b, kk * b_step),
                         idesc, (kb > kb_begin || kk != 0) ? 1u : 0u);
          umma_commit(empty_bar(stage));  // the stage may be refilled once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(acc_full_bar(buffer));
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quadrant = warp & 3;  // TMEM lanes [32*quadrant, 32*quadrant+32) are the ones this warp may read
    int local_tile = 0;
    bool ok = true;
    for (int work = blockIdx.x; ok && work < work_items; work += gridDim.x, ++local_tile) {
      const TileCoord coord = tile_coord(work % tiles, m_blocks, n_blocks, group_m);
      const int buffer = local_tile & 1;
      const uint32_t acc_phase = (uint32_t)(local_tile >> 1) & 1u;
      ok = mbar_wait(acc_full_bar(buffer), acc_phase, abort_flag, status_word, kWaitAccFull);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective: leave together or not at all
      if (!ok) break;
      tcgen05_fence_after();
      const int col0 = coord.n_block * TN;
      const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)(buffer * ACC_COLUMNS);
      store_accumulator_rows<OutT, TN>(dst, taddr, coord.m_block * BM + quadrant * 32, lane, m, n, col0,
                                   smem_aligned + STAGES * STAGE_BYTES + 256 + (warp - 2) * STAGING_BYTES_PER_WARP,
                                   (work / tiles) * m);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(buffer));
    }
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // a wait was abandoned: give copies that may still be in flight a bounded time to land before the
    // shared memory and TMEM are released
    const unsigned long long started = global_timer_ns();
    while (global_timer_ns() - started < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLUMNS);
  }
}

// Folds the fp32 partial products of a K-split GEMM — `partial` is [splits * m, n], one row block per split —
// into C (every destination of the gather form), rounding once.
template <typename OutT>
__global__ void __launch_bounds__(256) split_k_fold_kernel(const float* __restrict__ partial, const __grid_constant__ Destinations dst,
                                                           int m, int n, int splits) {
  const size_t total = (size_t)m * n;
  const size_t slice = total;  // elements per split
  if ((n & 3) == 0) {
    const size_t index = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (index >= total) return;
    float4 sum = *reinterpret_cast<const float4*>(partial + index);
    for (int s = 1; s < splits; ++s) {
      const float4 part = *reinterpret_cast<const float4*>(partial + (size_t)s * slice + index);
      sum.x += part.x; sum.y += part.y; sum.z += part.z; sum.w += part.w;
    }
    const size_t out_index = index + (size_t)dst.row_offset * n;
    for (int d = 0; d < dst.count; ++d) {
      OutT* out = static_cast<OutT*>(dst.p[d]) + out_index;
      if constexpr (sizeof(OutT) == 2) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
        if ((reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
          *reinterpret_cast<uint2*>(out) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        } else {
          out[0] = lo.x; out[1] = lo.y; out[2] = hi.x; out[3] = hi.y;
        }
      } else {
        if ((reinterpret_cast<uintptr_t>(out) & 15u) == 0) *reinterpret_cast<float4*>(out) = sum;
        else { out[0] = sum.x; out[1] = sum.y; out[2] = sum.z; out[3] = sum.w; }
      }
    }
  } else {
    for (size_t index = (size_t)blockIdx.x * blockDim.x * 4 + threadIdx.x; index < total && index < ((size_t)blockIdx.x + 1) * blockDim.x * 4;
         index += blockDim.x) {
      float sum = partial[index];
      for (int s = 1; s < splits; ++s) sum += partial[(size_t)s * slice + index];
      const size_t out_index = index + (size_t)dst.row_offset * n;
      for (int d = 0; d < dst.count; ++d) {
        if constexpr (sizeof(OutT) == 2) static_cast<__nv_bfloat16*>(dst.p[d])[out_index] = __float2bfloat16_rn(sum);
        else static_cast<float*>(dst.p[d])[out_index] = sum;
      }
    }
  }
}

// ---- CTA-pair variant ----------------------------------------------------------------------------------
// Two CTAs of a cluster (neighbouring SMs) own one 256x256 tile of C.  Each CTA streams its own 128
// rows of A and its own half (128 of the 256 n) of the B tile, so a stage is 32 KB instead of 48 KB and the
// ring holds 6 stages; CTA 0 issues tcgen05.mma.cta_group::2 (M256 x N256 x K16), which reads A from
// each CTA's shared memory, B from both halves, and writes each CTA's 128 accumulator lanes in that
// CTA's TMEM.  Per k-block the pair moves 64 KB for 8.4 MFLOP: a third less shared-memory and L2
// traffic per flop than the single-CTA kernel.
//   * TMA loads of both CTAs credit CTA 0's `full[stage]`, which expects the bytes of both.
//   * tcgen05.commit arrives on `empty[stage]` / `acc_full[buffer]` of BOTH CTAs (each CTA's producer
//     and epilogue wait on their own copy).
//   * the epilogue warps of both CTAs arrive on CTA 0's `acc_empty[buffer]` (8 arrivals).
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_ROWS = BN / 2;                       // rows of the B tile held by each CTA
constexpr int PAIR_B_BYTES = PAIR_B_ROWS * BK * 2;        // 16 KB
constexpr int PAIR_STAGE_BYTES = A_TILE_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 + STAGING_BYTES;
constexpr int PAIR_BM = 2 * BM;

template <typename OutT, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_abt_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ Destinations dst,
                     int m, int n, int k, int group_m, int* status_word) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_addr(smem_raw));
  uint64_t* barriers = reinterpret_cast<uint64_t*>(smem_aligned + PAIR_STAGES * PAIR_STAGE_BYTES);
  const uint32_t bar_base = smem_base + PAIR_STAGES * PAIR_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (PAIR_STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * PAIR_STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * PAIR_STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(barriers + 2 * PAIR_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_blocks = (m + PAIR_BM - 1) / PAIR_BM, n_blocks = (n + BN - 1) / BN;
  const int tiles = m_blocks * n_blocks;
  const int k_blocks = (k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 8);  // one arrival per epilogue warp of either CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  // the peer's barriers must exist before anything of this CTA can signal them
  cluster_arrive();
  cluster_wait();
  if (warp == 1) tmem_alloc_pair(smem_addr(tmem_slot), TMEM_COLUMNS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (elect_one()) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles; tile += pairs) {
        const TileCoord coord = tile_coord(tile, m_blocks, n_blocks, group_m);
        const int a_row = coord.m_block * PAIR_BM + (int)cta_rank * BM;
        const int b_row = coord.n_block * BN + (int)cta_rank * PAIR_B_ROWS;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status_word, kWaitEmpty))) break;
          const uint32_t a_dst = smem_base + stage * PAIR_STAGE_BYTES;
          const uint32_t signal = leader_cta_address(full_bar(stage));
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * PAIR_STAGE_BYTES);
          if constexpr (A_MN) {
#pragma unroll
            for (int t = 0; t < BM / 64; ++t)
              tma_load_2d_pair(a_dst + t * (BK * 128), &map_a, signal, a_row + t * 64, kb * BK);
          } else {
            tma_load_2d_pair(a_dst, &map_a, signal, kb * BK, a_row);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int t = 0; t < PAIR_B_ROWS / 64; ++t)
              tma_load_2d_pair(a_dst + A_TILE_BYTES + t * (BK * 128), &map_b, signal, b_row + t * 64, kb * BK);
          } else {
            tma_load_2d_pair(a_dst + A_TILE_BYTES, &map_b, signal, kb * BK, b_row);
          }
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (CTA 0 only) ----------------
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(PAIR_BM, BN, A_MN, B_MN);
      constexpr uint32_t a_step = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t b_step = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles; tile += pairs, ++local_tile) {
        const int buffer = local_tile & 1;
        const uint32_t acc_phase = (uint32_t)(local_tile >> 1) & 1u;
        if (!(ok = mbar_wait(acc_empty_bar(buffer), acc_phase ^ 1u, abort_flag, status_word, kWaitAccEmpty))) break;
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buffer * ACC_COLUMNS);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, status_word, kWaitFull))) break;
          tcgen05_fence_after();
          const uint32_t a_src = smem_base + stage * PAIR_STAGE_BYTES;
          const uint64_t desc_a = A_MN ? umma_desc_mn_major_sw128(a_src, BK * 128) : umma_desc_k_major_sw128(a_src);
          const uint64_t desc_b = B_MN ? umma_desc_mn_major_sw128(a_src + A_TILE_BYTES, BK * 128)
                                       : umma_desc_k_major_sw128(a_src + A_TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_bf16_ss_pair(tmem_acc, umma_desc_advance_k(desc_a, kk * a_step), umma_desc_advance_k(desc_b, kk * b_step),
                              idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit_pair(empty_bar(stage), 0x3);
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(acc_full_bar(buffer), 0x3);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs; each CTA stores its own 128 rows) ----------------
    const int quadrant = warp & 3;
    int local_tile = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < tiles; tile += pairs, ++local_tile) {
      const TileCoord coord = tile_coord(tile, m_blocks, n_blocks, group_m);
      const int buffer = local_tile & 1;
      const uint32_t acc_phase = (uint32_t)(local_tile >> 1) & 1u;
      ok = mbar_wait(acc_full_bar(buffer), acc_phase, abort_flag, status_word, kWaitAccFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int col0 = coord.n_block * BN;
      const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)(buffer * ACC_COLUMNS);
      store_accumulator_rows<OutT, BN>(dst, taddr, coord.m_block * PAIR_BM + (int)cta_rank * BM + quadrant * 32, lane, m, n, col0,
                                   smem_aligned + PAIR_STAGES * PAIR_STAGE_BYTES + 256 + (warp - 2) * STAGING_BYTES_PER_WARP);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty_bar(buffer), 0);
    }
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long started = global_timer_ns();
    while (global_timer_ns() - started < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may release its TMEM or shared memory while the other can still signal or read it;
  // every wait above is bounded, so both CTAs get here
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLUMNS);
  }
}

// ---- wide CTA-pair kernel: 512 x 256 tiles, K-major operands ------------------------------------------
// The same pair structure with each CTA holding TWO 128-row blocks of A per stage (256 rows) next to its half
// of the B tile: per k-block a pair moves 96 KB for 16.8 MFLOP — a quarter less shared-memory fill and L2 traffic per
// flop than the 256 x 256 pair tile, which under the power cap is worth more clock than anything else left in this
// kernel (measured on one box against the library GEMM, which uses this tile: 9.6 GB against 5.4 GB through L2 per
// 8192^3 product, tensor pipe 98 % against 96 % busy, SM clock 1.37 against 1.47 GHz).  The two accumulators of a CTA
// (rows 0-127 and 128-255 of its 256) take all 512 TMEM columns, so the epilogue of a tile is not hidden behind the
// next tile's MMAs as in the narrower kernels — about 3 % of a tile's time — while the producer keeps prefetching.
// CTA c of the pair owns rows [c*256, c*256 + 256) of the tile; MMA h of a k-step multiplies row block h of both CTAs.
constexpr int WIDE_STAGES = 4;
constexpr int WIDE_THREADS = 64 + 8 * 32;  // TMA warp, MMA warp, eight epilogue warps (one per accumulator and lane quadrant)

// One warp's 32 rows x 256 columns of one accumulator straight from registers into the single local C: a lane owns a
// row and writes it 64 bytes (bf16) or 128 bytes (f32) at a time while the next 32 columns are already on their way
// out of TMEM.  No staging: the wide kernel's shared memory is all ring, and local L2 merges the 16-byte pieces.
template <typename OutT>
__device__ __forceinline__ void store_accumulator_rows_direct(OutT* c, uint32_t taddr, int row, int m, int n, int col0) {
  constexpr int CHUNKS = BN / 32;
  uint32_t acc[2][32];
  tmem_ld_32x32b_x32(taddr, acc[0]);
#pragma unroll
  for (int chunk = 0; chunk < CHUNKS; ++chunk) {
    tmem_ld_wait();
    if (chunk + 1 < CHUNKS) tmem_ld_32x32b_x32(taddr + (uint32_t)((chunk + 1) * 32), acc[(chunk + 1) & 1]);
    const int col = col0 + chunk * 32;
    if (row < m && col < n) store_chunk<OutT>(c + (size_t)row * n + col, acc[chunk & 1], n - col);
  }
}
constexpr int WIDE_A_BYTES = 2 * A_TILE_BYTES;                 // 32 KB: two [128, 64] blocks
constexpr int WIDE_STAGE_BYTES = WIDE_A_BYTES + PAIR_B_BYTES;  // 48 KB
constexpr int WIDE_SMEM_BYTES = WIDE_STAGES * WIDE_STAGE_BYTES + 1024 + 256;
constexpr int WIDE_BM = 4 * BM;                                // 512 rows per pair tile

// bf16 output: the whole 256-column row of a lane fits in 128 registers once it is rounded, so the accumulator can be
// read out completely — and handed back to the MMA issuer — BEFORE the first global store is issued; the stores then
// drain underneath the next tile's MMAs.  (The stores, not the TMEM reads, are what an exposed epilogue costs: with the
// stores taken out the kernel ran 5 % faster, with the reads taken out no faster.)
__device__ __forceinline__ void load_row_packed_bf16(uint32_t taddr, uint32_t (&packed)[BN / 2]) {
  // 16 columns at a time, two loads in flight: 32 transient registers next to the 128 that hold the rounded row
  constexpr int CHUNKS = BN / 16;
  uint32_t acc[2][16];
  tmem_ld_32x32b_x16(taddr, acc[0]);
#pragma unroll
  for (int chunk = 0; chunk < CHUNKS; ++chunk) {
    tmem_ld_wait();
    if (chunk + 1 < CHUNKS) tmem_ld_32x32b_x16(taddr + (uint32_t)((chunk + 1) * 16), acc[(chunk + 1) & 1]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(acc[chunk & 1][2 * j]), __uint_as_float(acc[chunk & 1][2 * j + 1]));
      packed[chunk * 8 + j] = *reinterpret_cast<const uint32_t*>(&pair);
    }
  }
}

// n is a multiple of 8 and C is 16-byte aligned here (the launcher sends other shapes to the narrower kernels), so a
// 16-byte piece is either whole or absent.
__device__ __forceinline__ void store_row_packed_bf16(__nv_bfloat16* c, int row, int m, int n, int col0, const uint32_t (&packed)[BN / 2]) {
  if (row >= m) return;
  uint4* row_ptr = reinterpret_cast<uint4*>(c + (size_t)row * n + col0);
#pragma unroll
  for (int piece = 0; piece < BN / 8; ++piece)
    if (col0 + piece * 8 < n) row_ptr[piece] = make_uint4(packed[piece * 4], packed[piece * 4 + 1], packed[piece * 4 + 2], packed[piece * 4 + 3]);
}

template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WIDE_THREADS, 1)
gemm_abt_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ Destinations dst,
                     int m, int n, int k, int group_m, int* status_word) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_addr(smem_raw));
  uint64_t* barriers = reinterpret_cast<uint64_t*>(smem_aligned + WIDE_STAGES * WIDE_STAGE_BYTES);
  const uint32_t bar_base = smem_base + WIDE_STAGES * WIDE_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (WIDE_STAGES + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (2 * WIDE_STAGES);
  const uint32_t acc_empty_bar = bar_base + 8u * (2 * WIDE_STAGES + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(barriers + 2 * WIDE_STAGES + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_blocks = (m + WIDE_BM - 1) / WIDE_BM, n_blocks = (n + BN - 1) / BN;
  const int tiles = m_blocks * n_blocks;
  const int k_blocks = (k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WIDE_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar, 1);
    mbar_init(acc_empty_bar, 16);  // one arrival per epilogue warp of either CTA
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  cluster_arrive();  // the peer's barriers must exist before anything of this CTA can signal them
  cluster_wait();
  if (warp == 1) tmem_alloc_pair(smem_addr(tmem_slot), TMEM_COLUMNS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (elect_one()) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles; tile += pairs) {
        const TileCoord coord = tile_coord(tile, m_blocks, n_blocks, group_m);
        const int a_row = coord.m_block * WIDE_BM + (int)cta_rank * (2 * BM);
        const int b_row = coord.n_block * BN + (int)cta_rank * PAIR_B_ROWS;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status_word, kWaitEmpty))) break;
          const uint32_t a_dst = smem_base + stage * WIDE_STAGE_BYTES;
          const uint32_t signal = leader_cta_address(full_bar(stage));
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * WIDE_STAGE_BYTES);
          tma_load_2d_pair(a_dst, &map_a, signal, kb * BK, a_row);
          tma_load_2d_pair(a_dst + A_TILE_BYTES, &map_a, signal, kb * BK, a_row + BM);
          tma_load_2d_pair(a_dst + WIDE_A_BYTES, &map_b, signal, kb * BK, b_row);
          if (++stage == WIDE_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (CTA 0 only) ----------------
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(PAIR_BM, BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles; tile += pairs, ++local_tile) {
        // both accumulators of both CTAs must have been read by the previous tile's epilogue
        if (!(ok = mbar_wait(acc_empty_bar, ((uint32_t)local_tile & 1u) ^ 1u, abort_flag, status_word, kWaitAccEmpty))) break;
        tcgen05_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, status_word, kWaitFull))) break;
          tcgen05_fence_after();
          const uint32_t a_src = smem_base + stage * WIDE_STAGE_BYTES;
          const uint64_t desc_a0 = umma_desc_k_major_sw128(a_src);
          const uint64_t desc_a1 = umma_desc_k_major_sw128(a_src + A_TILE_BYTES);
          const uint64_t desc_b = umma_desc_k_major_sw128(a_src + WIDE_A_BYTES);
          // the four k-steps of one accumulator back to back, then the other's: consecutive MMAs into the same
          // accumulator chain inside the tensor core, alternating accumulators every instruction does not
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_bf16_ss_pair(tmem_base + (uint32_t)(half * ACC_COLUMNS), umma_desc_advance_k(half ? desc_a1 : desc_a0, kk * UMMA_K * 2),
                                umma_desc_advance_k(desc_b, kk * UMMA_K * 2), idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit_pair(empty_bar(stage), 0x3);
          if (++stage == WIDE_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(acc_full_bar, 0x3);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9 of both CTAs; warp = one lane quadrant of one accumulator) ----------------
    const int quadrant = warp & 3;          // TMEM lanes [32*quadrant, +32) are the ones this warp may touch
    const int half = (warp - 2) >> 2;       // which of the CTA's two accumulators (row blocks)
    OutT* c = static_cast<OutT*>(dst.p[0]) + (size_t)dst.row_offset * n;
    int local_tile = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < tiles; tile += pairs, ++local_tile) {
      const TileCoord coord = tile_coord(tile, m_blocks, n_blocks, group_m);
      ok = mbar_wait(acc_full_bar, (uint32_t)local_tile & 1u, abort_flag, status_word, kWaitAccFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)(half * ACC_COLUMNS);
      const int row = coord.m_block * WIDE_BM + (int)cta_rank * (2 * BM) + half * BM + quadrant * 32 + lane;
      if constexpr (sizeof(OutT) == 2) {
        uint32_t packed[BN / 2];
        load_row_packed_bf16(taddr, packed);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(acc_empty_bar, 0);  // the accumulator is in registers: the next tile may start
        store_row_packed_bf16(c, row, m, n, coord.n_block * BN, packed);
      } else {
        store_accumulator_rows_direct<OutT>(c, taddr, row, m, n, coord.n_block * BN);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(acc_empty_bar, 0);
      }
    }
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long started = global_timer_ns();
    while (global_timer_ns() - started < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_arrive();  // neither CTA may release its TMEM or shared memory while the other can still signal or read it
  cluster_wait();
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLUMNS);
  }
}

// ---- tiled transpose (brings other operand layouts to the native K-contiguous form) ------------------
__global__ void transpose_bf16_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int rows, int cols) {
  __shared__ __nv_bfloat16 tile[32][33];
  // tiles are numbered along grid.x alone (2^31 - 1 blocks): a long, narrow matrix must not run into the 65535 limit of grid.y
  const unsigned tiles_across = (unsigned)(cols + 31) / 32;
  const int c0 = (int)(blockIdx.x % tiles_across) * 32, r0 = (int)(blockIdx.x / tiles_across) * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[(size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[threadIdx.x][j];
  }
}

int launch_transpose(const void* src, void* dst, int rows, int cols, cudaStream_t stream) {
  const unsigned long long tiles = (unsigned long long)((cols + 31) / 32) * (unsigned long long)((rows + 31) / 32);
  if (tiles > 0x7fffffffull) return fail(BB200_E_UNSUPPORTED_SHAPE, "transpose: %d x %d needs more than 2^31 - 1 tiles", rows, cols);
  dim3 grid((unsigned)tiles), block(32, 8);
  transpose_bf16_kernel<<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols);
  return check_launch("transpose kernel launch");
}

constexpr int kMaxDevices = 64;

int current_device() {
  int device = 0;
  return cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < kMaxDevices ? device : -1;
}

// Host-side caches below are atomics or initialised-once statics: entry points may be called from several threads.
int cached_sm_count(int device) {
  static std::atomic<int> counts[kMaxDevices];
  int count = counts[device].load(std::memory_order_relaxed);
  if (count == 0) {
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) count = 0;
    counts[device].store(count, std::memory_order_relaxed);
  }
  return count;
}

// Tiles that run concurrently (148 consecutive tile ids) cover group_m M-blocks x 148/group_m N-blocks;
// 16 keeps that footprint (A rows + B rows of one wave) inside the 126 MB L2 for K up to 8192.
// BB200_GEMM_GROUP_M overrides it for tuning runs.
int raster_group_m() {
  static const int value = [] {
    const char* text = getenv("BB200_GEMM_GROUP_M");
    const int parsed = text ? atoi(text) : 0;
    return parsed > 0 && parsed <= 1024 ? parsed : DEFAULT_GROUP_M;
  }();
  return value;
}

// The pair kernel pays off once there are 256x256 tiles for at least half of the CTA pairs (a pair tile streams a third
// less per flop, so even a half-occupied wave beats single-CTA tiles at full occupancy); smaller and ragged
// problems stay on the single-CTA kernel.  BB200_GEMM_PAIR=0/1 forces the choice for tuning runs.
bool use_pair_kernel(int m, int n, int sms) {
  static const int forced = [] {
    const char* text = getenv("BB200_GEMM_PAIR");
    return text ? (atoi(text) != 0 ? 1 : 0) : -1;  // 1 and 2 (the wide tile) both mean a CTA-pair kernel
  }();
  if (forced >= 0) return forced == 1;
  const long tiles = (long)((m + PAIR_BM - 1) / PAIR_BM) * ((n + BN - 1) / BN);
  // an odd number of 128-row blocks leaves the last pair tile half empty: tolerable from nine blocks on
  const int m_blocks = (m + BM - 1) / BM;
  const bool rows_fill_pairs = (m_blocks % 2) == 0 || m_blocks >= 9;
  return (sms % 2) == 0 && rows_fill_pairs && tiles >= sms / 4;
}

template <typename OutT, bool A_MN, bool B_MN>
int launch_pair(const void* a_operand, const void* b, const Destinations& dst, int m, int n, int k, int device, int sms, cudaStream_t stream) {
  alignas(64) CUtensorMap map_a, map_b;
  if (int status = A_MN ? encode_tensormap_2d(&map_a, BB200_BF16, a_operand, (uint64_t)k, (uint64_t)m, (uint64_t)m * 2, BK, 64, 3)
                        : encode_tensormap_2d(&map_a, BB200_BF16, a_operand, (uint64_t)m, (uint64_t)k, (uint64_t)k * 2, BM, BK, 3))
    return status;
  if (int status = B_MN ? encode_tensormap_2d(&map_b, BB200_BF16, b, (uint64_t)k, (uint64_t)n, (uint64_t)n * 2, BK, 64, 3)
                        : encode_tensormap_2d(&map_b, BB200_BF16, b, (uint64_t)n, (uint64_t)k, (uint64_t)k * 2, PAIR_B_ROWS, BK, 3))
    return status;
  static std::atomic<bool> configured[kMaxDevices];
  if (!configured[device]) {
    if (int status = check_runtime(cudaFuncSetAttribute(gemm_abt_pair_kernel<OutT, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES),
                                   "cudaFuncSetAttribute(gemm pair smem)"))
      return status;
    configured[device] = true;
  }
  const int tiles = ((m + PAIR_BM - 1) / PAIR_BM) * ((n + BN - 1) / BN);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  gemm_abt_pair_kernel<OutT, A_MN, B_MN><<<2 * pairs, THREADS, PAIR_SMEM_BYTES, stream>>>(map_a, map_b, dst, m, n, k, raster_group_m() / 2 > 0 ? raster_group_m() / 2 : 1,
                                                                             device_status_word());
  return check_launch("gemm pair kernel launch");
}

template <typename OutT>
int launch_wide(const void* a, const void* b, const Destinations& dst, int m, int n, int k, int device, int sms, cudaStream_t stream) {
  alignas(64) CUtensorMap map_a, map_b;
  if (int status = encode_tensormap_2d(&map_a, BB200_BF16, a, (uint64_t)m, (uint64_t)k, (uint64_t)k * 2, BM, BK, 3)) return status;
  if (int status = encode_tensormap_2d(&map_b, BB200_BF16, b, (uint64_t)n, (uint64_t)k, (uint64_t)k * 2, PAIR_B_ROWS, BK, 3)) return status;
  static std::atomic<bool> configured[kMaxDevices];
  if (!configured[device]) {
    if (int status = check_runtime(cudaFuncSetAttribute(gemm_abt_wide_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, WIDE_SMEM_BYTES),
                                   "cudaFuncSetAttribute(gemm wide smem)"))
      return status;
    configured[device] = true;
  }
  const int tiles = ((m + WIDE_BM - 1) / WIDE_BM) * ((n + BN - 1) / BN);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  // eight 512-row bands per raster group: measured best at 8192^3 (group 4 / 6 / 8 / 10 / 12 bands: 1614 / 1617 / 1622 /
  // 1608 / 1605 TFLOP/s on one box) — a wave of 74 tiles then spans 9 column blocks, and A (64 MB) stays in L2 with them
  const int group = raster_group_m() / 2 > 0 ? raster_group_m() / 2 : 1;
  gemm_abt_wide_kernel<OutT><<<2 * pairs, WIDE_THREADS, WIDE_SMEM_BYTES, stream>>>(map_a, map_b, dst, m, n, k, group, device_status_word());
  return check_launch("gemm wide kernel launch");
}

// The wide tile wins whenever it wastes no more of the machine than the 256-row pair tile does: the fraction of tile
// area inside the matrix times the fraction of the last wave that is occupied, with a few per cent of credit for the
// lower traffic.  BB200_GEMM_PAIR=2 forces it, 1 forces the 256-row pair tile (tuning and tests).
bool use_wide_kernel(int m, int n, int k, int sms) {
  static const int forced = [] {
    const char* text = getenv("BB200_GEMM_PAIR");
    return text ? atoi(text) : -1;
  }();
  if (forced == 2) return true;
  if (forced >= 0) return false;
  auto efficiency = [&](int tile_rows) {
    const long m_blocks = (m + tile_rows - 1) / tile_rows, n_blocks = (n + BN - 1) / BN;
    const long tiles = m_blocks * n_blocks, pairs = sms / 2;
    const long waves = (tiles + pairs - 1) / pairs;
    return ((double)m * n / ((double)m_blocks * tile_rows * n_blocks * BN)) * ((double)tiles / (double)(waves * pairs));
  };
  // Both accumulators of a CTA belong to one tile, so the read-out of a tile is not hidden behind the next tile's products
  // as in the narrower kernels: the wide tile pays off only when the products of a tile are long enough (measured at
  // 8192 x 8192 x K, one cold launch each: K = 1024 / 2048 / 4096 117 / 183 / 335 us against 102 / 164 / 328 for the 256-row
  // tile, K = 6144 / 8192 504 / 654 against 510 / 678).
  return k >= 6144 && m >= WIDE_BM && efficiency(WIDE_BM) * 1.03 >= efficiency(PAIR_BM);
}

// A_MN: A is stored [k, m] (m contiguous) and consumed as an MN-major operand; otherwise [m, k].
// B_MN: B is stored [k, n] (n contiguous), MN-major; otherwise [n, k].
// Tile width of the single-CTA kernel.  BB200_GEMM_TILE_N = 256 / 128 / 64 forces it for tuning runs.
int single_cta_tile_n(int m, int n, int sms) {
  static const int forced = [] {
    const char* text = getenv("BB200_GEMM_TILE_N");
    const int parsed = text ? atoi(text) : 0;
    return parsed == 256 || parsed == 128 || parsed == 64 ? parsed : 0;
  }();
  if (forced) return forced;
  // a wave of full-width tiles that (nearly) fills the SMs stays; otherwise the narrowest width whose tiles still fit one
  // wave: a lone tile is bound by the latency of its own operand stream, and narrower tiles put more streams in flight
  const long m_blocks = (m + BM - 1) / BM;
  if (m_blocks * ((n + 255) / 256) * 10 >= (long)sms * 9) return 256;
  int chosen = 256;
  for (int width : {128, 64}) {
    if (m_blocks * ((n + width - 1) / width) <= (long)sms) chosen = width;
  }
  return chosen;
}

Destinations single_destination(void* c) {
  Destinations dst = {};
  dst.p[0] = c;
  dst.count = 1;
  dst.row_offset = 0;
  return dst;
}

// K-splits of the single-CTA kernel: when even the narrowest tiles leave most SMs idle and K is deep, each tile's K
// range is cut into `splits` work items whose fp32 partial products a second kernel folds.  Needs a workspace, so the
// allocation-free entry point never splits.  BB200_GEMM_SPLIT_K forces a count (1 = never) for tuning runs.
int split_k_count(int tiles, int k_blocks, int sms) {
  static const int forced = [] {
    const char* text = getenv("BB200_GEMM_SPLIT_K");
    const int parsed = text ? atoi(text) : 0;
    return parsed >= 1 && parsed <= 64 ? parsed : 0;
  }();
  int splits = forced ? forced : (tiles * 2 <= sms ? sms / tiles : 1);
  if (splits > 16 && !forced) splits = 16;
  if (splits > k_blocks / 8) splits = k_blocks / 8;  // at least eight 64-wide k-blocks per work item
  return splits < 2 ? 1 : splits;
}

// Split-K workspaces come from a pool of this library's own that keeps what is freed (release threshold = everything):
// the device's default pool hands memory back at every synchronisation, and a caller that synchronises between two GEMMs
// would then pay a fresh allocation (≈ 130 us) for every call.
cudaMemPool_t workspace_pool(int device) {
  static std::mutex guard;
  static cudaMemPool_t pools[kMaxDevices] = {};
  std::lock_guard<std::mutex> lock(guard);
  if (!pools[device]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    cudaMemPool_t created = nullptr;
    if (cudaMemPoolCreate(&created, &props) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    unsigned long long keep_everything = ~0ull;
    cudaMemPoolSetAttribute(created, cudaMemPoolAttrReleaseThreshold, &keep_everything);
    pools[device] = created;
  }
  return pools[device];
}

template <typename OutT, bool A_MN, bool B_MN, int TN>
int launch_single(const void* a_operand, const void* b, const Destinations& dst, int m, int n, int k, int device, int sms, bool may_split,
                  cudaStream_t stream) {
  using T = Tile<TN>;
  alignas(64) CUtensorMap map_a, map_b;
  if (int status = A_MN ? encode_tensormap_2d(&map_a, BB200_BF16, a_operand, (uint64_t)k, (uint64_t)m, (uint64_t)m * 2, BK, 64, 3)
                        : encode_tensormap_2d(&map_a, BB200_BF16, a_operand, (uint64_t)m, (uint64_t)k, (uint64_t)k * 2, BM, BK, 3))
    return status;
  if (int status = B_MN ? encode_tensormap_2d(&map_b, BB200_BF16, b, (uint64_t)k, (uint64_t)n, (uint64_t)n * 2, BK, 64, 3)
                        : encode_tensormap_2d(&map_b, BB200_BF16, b, (uint64_t)n, (uint64_t)k, (uint64_t)k * 2, TN, BK, 3))
    return status;
  static std::atomic<bool> configured[kMaxDevices];  // per template instantiation and device
  if (!configured[device]) {
    if (int status = check_runtime(cudaFuncSetAttribute(gemm_abt_kernel<OutT, A_MN, B_MN, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES),
                                   "cudaFuncSetAttribute(gemm smem)"))
      return status;
    if (int status = check_runtime(cudaFuncSetAttribute(gemm_abt_kernel<float, A_MN, B_MN, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES),
                                   "cudaFuncSetAttribute(gemm smem)"))
      return status;
    configured[device] = true;
  }
  const int tiles = ((m + BM - 1) / BM) * ((n + TN - 1) / TN);
  const int k_blocks = (k + BK - 1) / BK;
  const int splits = may_split ? split_k_count(tiles, k_blocks, sms) : 1;
  if (splits > 1) {
    const int kb_per_split = (k_blocks + splits - 1) / splits;
    const int used_splits = (k_blocks + kb_per_split - 1) / kb_per_split;  // no empty K ranges
    float* partial = nullptr;
    cudaMemPool_t pool = workspace_pool(device);
    if (!pool) return fail(BB200_E_NO_DRIVER, "gemm: could not create the split-K workspace pool");
    if (int status = check_runtime(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&partial), (size_t)used_splits * m * n * sizeof(float), pool, stream),
                                   "cudaMallocFromPoolAsync(gemm split-K workspace)"))
      return status;
    const Destinations workspace = single_destination(partial);
    const int work_items = tiles * used_splits;
    gemm_abt_kernel<float, A_MN, B_MN, TN><<<work_items < sms ? work_items : sms, THREADS, T::SMEM_BYTES, stream>>>(
        map_a, map_b, workspace, m, n, k, raster_group_m(), used_splits, kb_per_split, device_status_word());
    int status = check_launch("gemm split-K kernel launch");
    if (!status) {
      const size_t quads = ((size_t)m * n + 3) / 4;
      split_k_fold_kernel<OutT><<<(unsigned)((quads + 255) / 256), 256, 0, stream>>>(partial, dst, m, n, used_splits);
      status = check_launch("gemm split-K fold launch");
    }
    const int freed = check_runtime(cudaFreeAsync(partial, stream), "cudaFreeAsync(gemm split-K workspace)");
    return status ? status : freed;
  }
  const int grid = tiles < sms ? tiles : sms;
  gemm_abt_kernel<OutT, A_MN, B_MN, TN><<<grid, THREADS, T::SMEM_BYTES, stream>>>(map_a, map_b, dst, m, n, k, raster_group_m(), 1, k_blocks,
                                                                              device_status_word());
  return check_launch("gemm kernel launch");
}

template <typename OutT, bool A_MN, bool B_MN>
int launch_native(const void* a_operand, const void* b, const Destinations& dst, int m, int n, int k, bool may_split, cudaStream_t stream) {
  const int device = current_device();
  if (device < 0) return fail(BB200_E_NO_DRIVER, "gemm: no CUDA device is current");
  const int sms = cached_sm_count(device);
  if (sms <= 0) return fail(BB200_E_NO_DRIVER, "gemm: could not query the SM count");
  if (use_pair_kernel(m, n, sms)) {
    if constexpr (!A_MN && !B_MN) {
      // the wide kernel writes one local C in whole 16-byte pieces
      if (dst.count == 1 && (n % 8) == 0 && aligned16(dst.p[0]) && use_wide_kernel(m, n, k, sms)) return launch_wide<OutT>(a_operand, b, dst, m, n, k, device, sms, stream);
    }
    return launch_pair<OutT, A_MN, B_MN>(a_operand, b, dst, m, n, k, device, sms, stream);
  }
  switch (single_cta_tile_n(m, n, sms)) {
    case 256: return launch_single<OutT, A_MN, B_MN, 256>(a_operand, b, dst, m, n, k, device, sms, may_split, stream);
    case 128: return launch_single<OutT, A_MN, B_MN, 128>(a_operand, b, dst, m, n, k, device, sms, may_split, stream);
    default: return launch_single<OutT, A_MN, B_MN, 64>(a_operand, b, dst, m, n, k, device, sms, may_split, stream);
  }
}

int dispatch_native(const void* a_operand, const void* b, const Destinations& dst, int m, int n, int k, bool a_is_km, bool b_is_kn,
                    bb200_dtype c_dtype, bool may_split, cudaStream_t s) {
#define BB200_GEMM_CASE(OUT, A_MN, B_MN) \
  if (a_is_km == A_MN && b_is_kn == B_MN) return launch_native<OUT, A_MN, B_MN>(a_operand, b, dst, m, n, k, may_split, s)
  if (c_dtype == BB200_BF16) {
    BB200_GEMM_CASE(__nv_bfloat16, false, false);
    BB200_GEMM_CASE(__nv_bfloat16, false, true);
    BB200_GEMM_CASE(__nv_bfloat16, true, false);
    BB200_GEMM_CASE(__nv_bfloat16, true, true);
  } else {
    BB200_GEMM_CASE(float, false, false);
    BB200_GEMM_CASE(float, false, true);
    BB200_GEMM_CASE(float, true, false);
    BB200_GEMM_CASE(float, true, true);
  }
#undef BB200_GEMM_CASE
  return fail(BB200_E_INVALID_ARGUMENT, "gemm: unreachable operand layout");
}

}  // namespace
}  // namespace bb200

using namespace bb200;

static int gemm_bf16_into(const void* a, const void* b, const Destinations& destinations, int m, int n, int k, int transpose_a,
                          int transpose_b, bb200_dtype c_dtype, void* stream) {
  if (!a || !b) return fail(BB200_E_INVALID_ARGUMENT, "gemm: null tensor pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(BB200_E_INVALID_ARGUMENT, "gemm: m, n, k must be > 0 (got %d, %d, %d)", m, n, k);
  if (c_dtype != BB200_BF16 && c_dtype != BB200_F32) return fail(BB200_E_INVALID_ARGUMENT, "gemm: C must be bf16 or f32");
  if (k % 8) return fail(BB200_E_UNSUPPORTED_SHAPE, "gemm: k=%d must be a multiple of 8 (16-byte rows for TMA)", k);
  if (!aligned16(a) || !aligned16(b)) return fail(BB200_E_MISALIGNED, "gemm: A and B must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Both operands are consumed in place in either layout (MN-major descriptors).  The one exception is A
  // stored [k, m] with m not a multiple of 8: its rows are not 16-byte multiples, which TMA needs, so it is
  // transposed into a workspace first.
  const bool b_is_kn = !transpose_b;
  if (b_is_kn && (n % 8)) return fail(BB200_E_UNSUPPORTED_SHAPE, "gemm: n=%d must be a multiple of 8 when B is stored [k, n]", n);
  const bool a_in_place = transpose_a && (m % 8) == 0;
  const void* a_operand = a;
  void* workspace = nullptr;
  if (transpose_a && !a_in_place) {  // stored [k, m] -> [m, k]
    if (int status = check_runtime(cudaMallocAsync(&workspace, (size_t)m * k * 2, s), "cudaMallocAsync(gemm workspace)")) return status;
    if (int status = launch_transpose(a, workspace, k, m, s)) {
      cudaFreeAsync(workspace, s);
      return status;
    }
    a_operand = workspace;
  }
  int status = dispatch_native(a_operand, b, destinations, m, n, k, a_in_place, b_is_kn, c_dtype, /*may_split=*/true, s);
  if (workspace) {
    const int freed = check_runtime(cudaFreeAsync(workspace, s), "cudaFreeAsync(gemm workspace)");
    if (!status) status = freed;
  }
  return status;
}

extern "C" int bb200_gemm_bf16(const void* a, const void* b, void* c, int m, int n, int k, int transpose_a, int transpose_b,
                               bb200_dtype c_dtype, void* stream) {
  if (!c) return fail(BB200_E_INVALID_ARGUMENT, "gemm: null tensor pointer");
  return gemm_bf16_into(a, b, single_destination(c), m, n, k, transpose_a, transpose_b, c_dtype, stream);
}

extern "C" int bb200_gemm_bf16_gather(const void* a, const void* b, void* const* c_destinations, int destination_count, int row_offset,
                                      int m, int n, int k, int transpose_a, int transpose_b, bb200_dtype c_dtype, void* stream) {
  if (!c_destinations || destination_count < 1 || destination_count > kMaxDestinations)
    return fail(BB200_E_INVALID_ARGUMENT, "gemm (gather): 1..%d destination buffers are needed (got %d)", kMaxDestinations, destination_count);
  if (row_offset < 0) return fail(BB200_E_INVALID_ARGUMENT, "gemm (gather): row_offset must be >= 0");
  Destinations destinations = {};
  for (int d = 0; d < destination_count; ++d) {
    if (!c_destinations[d]) return fail(BB200_E_INVALID_ARGUMENT, "gemm (gather): destination %d is null", d);
    destinations.p[d] = c_destinations[d];
  }
  destinations.count = destination_count;
  destinations.row_offset = row_offset;
  return gemm_bf16_into(a, b, destinations, m, n, k, transpose_a, transpose_b, c_dtype, stream);
}

// ---- allocation-free variant -------------------------------------------------------------------------
// bb200_gemm_bf16 above borrows a stream-ordered workspace (cudaMallocAsync) whenever A arrives stored
// [k, m] with m not a multiple of 8 (the one layout TMA cannot read in place).  That is a problem for embedders that must not allocate while they run: an inference server
// that has already sized its own pools to fill the device (so a late driver allocation can fail or
// evict), a host framework whose caching allocator is meant to be the only owner of device memory, or
// a latency-critical loop where an allocation call may stall behind other work on the device.  For
// them the transposed copy of A goes into the fixed buffer below, which is part of the library image.
//
// The buffer is one per GPU for the life of the process (every device that loads this library holds
// these 32 MiB until exit).  It is shared by every call: calls whose GPU work can overlap (different
// streams, different host threads) would overwrite each other's copy of A — callers serialise them.
// Nothing in the buffer has to start at zero: each call rewrites the m*k elements it then reads.
constexpr size_t kGemmStaticScratchBytes = 32u << 20;  // transposed A of up to 16 Mi bf16 elements
static __device__ __align__(256) unsigned char g_gemm_static_scratch[kGemmStaticScratchBytes];

namespace {

// In host code `g_gemm_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use is looked up once per device, with that device current.
int gemm_static_scratch(void** device_ptr_out) {
  static void* resolved[64] = {};
  static std::mutex guard;
  int device = 0;
  if (int status = check_runtime(cudaGetDevice(&device), "cudaGetDevice")) return status;
  if (device < 0 || device >= 64) return fail(BB200_E_UNSUPPORTED_SHAPE, "gemm (no-alloc): device ordinal %d is out of range", device);
  std::lock_guard<std::mutex> lock(guard);
  if (!resolved[device]) {
    void* address = nullptr;
    if (int status = check_runtime(cudaGetSymbolAddress(&address, g_gemm_static_scratch),
                                   "cudaGetSymbolAddress(gemm static scratch)"))
      return status;
    if (!address) return fail(BB200_E_NO_DRIVER, "gemm (no-alloc): the static scratch buffer has no device address");
    resolved[device] = address;
  }
  *device_ptr_out = resolved[device];
  return BB200_OK;
}

}  // namespace

extern "C" int bb200_gemm_bf16_noalloc(const void* a, const void* b, void* c, int m, int n, int k, int transpose_a,
                                       int transpose_b, bb200_dtype c_dtype, void* stream) {
  if (!a || !b || !c) return fail(BB200_E_INVALID_ARGUMENT, "gemm (no-alloc): null tensor pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(BB200_E_INVALID_ARGUMENT, "gemm (no-alloc): m, n, k must be > 0 (got %d, %d, %d)", m, n, k);
  if (c_dtype != BB200_BF16 && c_dtype != BB200_F32) return fail(BB200_E_INVALID_ARGUMENT, "gemm (no-alloc): C must be bf16 or f32");
  if (k % 8) return fail(BB200_E_UNSUPPORTED_SHAPE, "gemm (no-alloc): k=%d must be a multiple of 8 (16-byte rows for TMA)", k);
  if (!aligned16(a) || !aligned16(b)) return fail(BB200_E_MISALIGNED, "gemm (no-alloc): A and B must be 16-byte aligned");
  const bool b_is_kn = !transpose_b;
  if (b_is_kn && (n % 8)) return fail(BB200_E_UNSUPPORTED_SHAPE, "gemm (no-alloc): n=%d must be a multiple of 8 when B is stored [k, n]", n);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool a_in_place = transpose_a && (m % 8) == 0;  // consumed as an MN-major operand: nothing to stage
  const void* a_operand = a;
  if (transpose_a && !a_in_place) {
    const size_t needed = (size_t)m * (size_t)k * 2;
    if (needed > kGemmStaticScratchBytes)
      return fail(BB200_E_TOO_LARGE,
                  "gemm (no-alloc): A stored [k, m] needs a %zu-byte transposed copy but the built-in buffer holds %zu bytes "
                  "(m*k <= %zu); pass A as [m, k], make m a multiple of 8, or use bb200_gemm_bf16",
                  needed, kGemmStaticScratchBytes, kGemmStaticScratchBytes / 2);
    void* scratch = nullptr;
    if (int status = gemm_static_scratch(&scratch)) return status;
    if (int status = launch_transpose(a, scratch, k, m, s)) return status;
    a_operand = scratch;
  }
  return dispatch_native(a_operand, b, single_destination(c), m, n, k, a_in_place, b_is_kn, c_dtype, /*may_split=*/false, s);
}

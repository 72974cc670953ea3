// attn_fwd_tcgen05.cu — softmax attention forward for sm_100a (bf16 in/out, fp32 online softmax).
//
//   out[b, q, h, :] = softmax_k( q·k / sqrt(D)  [masked to k <= q when causal] ) · v,   lse = ln Σ exp(...)
//
// Tensors are [batch, seq, heads, head_dim] row-major, so one (batch, head) slice is a matrix whose
// rows are `heads*head_dim` elements apart; TMA reads it through a 3-D map (head_dim*heads, seq,
// batch) and zero-fills rows past `seq`.
//
// A work item is TWO 128-query tiles of one (batch, head), for which the key/value blocks of 128 keys
// are walked once (only blocks at or below the diagonal when causal).  The kernel is persistent: one CTA
// per SM draws items from a counter in global memory until none is left.  384 threads in three
// warpgroups; warpgroup 0 gives registers back (setmaxnreg) so the softmax warpgroups can hold a
// full 128-column score row per thread:
//   warp 0       work distributor and TMA producer: fetches the next item, hands it to the other warps
//                through a two-slot ring, loads both Q tiles, then K and V blocks into a 2-stage ring.
//   warp 1       MMA issuer (one elected thread).  Per tile t and block j:  S_t = Q_t·K_j^T  into TMEM
//                (both operands K-major in shared memory), later  O_t += P_t·V_j  with P_t read from
//                TMEM and V_j consumed in place as an MN-major shared-memory operand.  The issue order
//                QK0, QK1, {PV0, QK0', PV1, QK1'}… keeps the tensor pipe busy with one tile while the
//                other tile's softmax runs.
//   warps 4..7   softmax of tile 0, warps 8..11 softmax of tile 1; thread = query row.  The fp32 score
//                row is read from TMEM once (128 registers), p = 2^(s·c − m·c) is written back over
//                the same TMEM columns as packed bf16, and the row sum is kept in fp32.  O stays in
//                TMEM for the whole walk; it is rescaled (tcgen05.ld / st) only when some row of the
//                warp sees its running maximum grow by more than 2^8, so most blocks skip it.
// TMEM (512 columns): S0/P0 [0,128), S1/P1 [128,256), O0 [256,256+D), O1 [384,384+D).
// Tensor-core bound (4·B·H·D·S(S+1)/2 flops causal); HBM traffic is ~4·B·S·H·D·2 bytes.
// Head dims other than 64/128 use a plain SIMT kernel below.
#include <cuda_bf16.h>
#include <math.h>

#include <atomic>

#include "bb200_internal.h"
#include "bb200_sm100.cuh"

namespace bb200 {
namespace {

using namespace sm100;

constexpr int BLOCK_M = 128, BLOCK_N = 128;
constexpr int Q_TILES = 2;                 // query tiles per CTA
constexpr int KV_STAGES = 2;
constexpr int THREADS = 128 * (1 + Q_TILES);  // warpgroup 0: TMA + MMA warps; warpgroups 1..2: softmax of tile 0 / 1
constexpr int SUBTILE_BYTES = 128 * 128;   // [128 rows, 64 bf16] with 128-byte rows
constexpr int DEFER_KEYS = 32;              // exponentials of the second half computed before the first half's store is awaited
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units: p stays below 2^8 between rescales

enum WaitCode { kWaitQ = 201, kWaitKvEmpty = 202, kWaitK = 203, kWaitV = 204, kWaitSReady = 205, kWaitPReady = 206,
                kWaitODone = 207, kWaitItem = 208, kWaitOFree = 209 };

template <int D> struct Smem {
  static constexpr int DCH = D / 64;                       // 64-column sub-tiles per row block
  static constexpr int Q_BYTES = DCH * SUBTILE_BYTES;      // one query tile
  static constexpr int K_BYTES = DCH * SUBTILE_BYTES;
  static constexpr int V_BYTES = DCH * SUBTILE_BYTES;
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = Q_OFF + Q_TILES * Q_BYTES;
  static constexpr int BAR_OFF = KV_OFF + KV_STAGES * (K_BYTES + V_BYTES);
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;       // barriers + alignment slack
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// max(a, b, c) in one instruction
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Where out and lse go.  Ordinarily one pair of tensors.  In the gather form this GPU's batches are a block of
// a larger batch of which every GPU of the box holds a copy: out rows and lse values are stored into all `count`
// copies (its own and, through peer-mapped pointers, the others') at batch `batch_offset + b`.
constexpr int kMaxDestinations = 8;
struct OutputDestinations {
  void* out[kMaxDestinations];
  float* lse[kMaxDestinations];
  int count;
  int batch_offset;
};

// GATHER = false: the single-destination kernel; each thread stores its own output row straight from registers.
// GATHER = true: rows are staged in the (by then unused) shared memory of the tile's Q and leave as whole
// contiguous rows, sixteen (or eight) lanes per row, into every destination — 16-byte pieces of 32 different rows
// per store instruction would waste most of an NVLink packet.
//
// The kernel is persistent: one CTA per SM takes work items — a pair of query tiles of one (batch, head) — from a
// counter in global memory until it runs dry, so the loads and the first Q·K^T of the next item overlap the last
// softmax, the epilogue and the stores of the current one, and TMEM, barriers and the register hand-over are set up
// once per SM.  Items are numbered (batch, head)-major with the longest causal pair first inside each (batch, head), so
// the CTAs that run together mostly share one head's keys and values in L2.  The producer warp fetches an item index
// and hands it to the other warps through a two-slot ring; every barrier parity follows running counters.
template <int D, bool CAUSAL, bool GATHER>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ OutputDestinations dst,
                int seq, int heads, int kv_heads, int batches, float scale_log2e, int* work_counter, int* status_word) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_addr(smem_raw));
  const uint32_t bar_base = base + L::BAR_OFF;
  // barriers: q_full, q_free, k_full[2], v_full[2], kv_empty[2], s_ready[2], p_ready[2 tiles][2 halves], o_done[2],
  // o_free[2], item_full[2], item_empty[2]
  const uint32_t q_full = bar_base, q_free = bar_base + 8u;
  auto k_full = [&](int s) { return bar_base + 8u * (2 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (4 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (6 + s); };
  auto s_ready = [&](int t) { return bar_base + 8u * (8 + t); };
  auto p_ready = [&](int t, int half) { return bar_base + 8u * (10 + 2 * t + half); };
  auto o_done = [&](int t) { return bar_base + 8u * (14 + t); };
  auto o_free = [&](int t) { return bar_base + 8u * (16 + t); };
  auto item_full = [&](int s) { return bar_base + 8u * (18 + s); };
  auto item_empty = [&](int s) { return bar_base + 8u * (20 + s); };
  constexpr int BARRIERS = 22;
  volatile int* item_slot = reinterpret_cast<volatile int*>(aligned + L::BAR_OFF + 8 * BARRIERS);  // two entries
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aligned + L::BAR_OFF + 8 * BARRIERS + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blocks = (seq + BLOCK_M - 1) / BLOCK_M;
  const int pairs = (q_blocks + Q_TILES - 1) / Q_TILES;
  const int kv_blocks_all = (seq + BLOCK_N - 1) / BLOCK_N;
  const int total_items = pairs * heads * batches;
  const int kv_group = heads / kv_heads;

  // a work item: which pair of query tiles of which (batch, head), and how many key/value blocks each tile needs
  struct Item {
    int pair, head, batch, blocks_of[Q_TILES], kv_blocks;
  };
  auto decode = [&](int index) {
    Item item;
    item.pair = pairs - 1 - index % pairs;  // longest causal rows first
    const int slice = index / pairs;
    item.head = slice % heads;
    item.batch = slice / heads;
#pragma unroll
    for (int t = 0; t < Q_TILES; ++t) {
      const int q_block = item.pair * Q_TILES + t;
      item.blocks_of[t] = q_block >= q_blocks ? 0 : (CAUSAL ? min(q_block + 1, kv_blocks_all) : kv_blocks_all);
    }
    item.kv_blocks = max(item.blocks_of[0], item.blocks_of[1]);
    return item;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, GATHER ? 1 + 2 * 4 : 1);  // the MMA issuer's commit, plus every softmax warp when Q doubles as staging
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int t = 0; t < Q_TILES; ++t) {
      mbar_init(s_ready(t), 1);
      mbar_init(p_ready(t, 0), 4);  // one arrival per softmax warp
      mbar_init(p_ready(t, 1), 4);
      mbar_init(o_done(t), 1);
      mbar_init(o_free(t), 4);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(item_full(s), 1);
      mbar_init(item_empty(s), 1 + 2 * 4);  // the MMA issuer and every softmax warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(smem_addr(tmem_slot), 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    // warpgroup 0 (TMA, MMA and two idle warps) hands registers to the softmax warpgroups.  64 + 216 leaves 2048
    // registers of the SM's file unclaimed; 80 + 216 claims all of it and the softmax warps' `inc` then never returns.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
  if (warp == 0) {
    // ---------------- TMA producer and work distributor ----------------
    if (elect_one()) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      bool ok = true;
      int kv_count = 0;  // key/value blocks loaded so far: ring stage and parity follow it across items
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        // the ring slot is free once the issuer and the softmax warps have finished the item before last
        if (!(ok = mbar_wait(item_empty(slot), ((uint32_t)(n >> 1) & 1u) ^ 1u, abort_flag, status_word, kWaitItem))) break;
        int index = atomicAdd(work_counter, 1);
        if (index >= total_items) index = -1;
        item_slot[slot] = index;
        mbar_arrive(item_full(slot));  // release: the slot is written before the arrival is seen
        if (index < 0) break;
        const Item item = decode(index);
        const int kv_head = item.head / kv_group;
        // Q may be overwritten once the previous item's last Q·K^T (and, in the gather form, its staged rows) are done
        if (!(ok = mbar_wait(q_free, ((uint32_t)n & 1u) ^ 1u, abort_flag, status_word, kWaitQ))) break;
        mbar_arrive_expect_tx(q_full, Q_TILES * L::Q_BYTES);
#pragma unroll
        for (int t = 0; t < Q_TILES; ++t)
#pragma unroll
          for (int c = 0; c < L::DCH; ++c)
            tma_load_3d(base + L::Q_OFF + t * L::Q_BYTES + c * SUBTILE_BYTES, &map_q, q_full, item.head * D + c * 64,
                        (item.pair * Q_TILES + t) * BLOCK_M, item.batch);
        for (int j = 0; ok && j < item.kv_blocks; ++j, ++kv_count) {
          const int stage = kv_count & 1;
          const uint32_t use_parity = (uint32_t)(kv_count >> 1) & 1u;
          if (!(ok = mbar_wait(kv_empty(stage), use_parity ^ 1u, abort_flag, status_word, kWaitKvEmpty))) break;
          const uint32_t k_dst = base + L::KV_OFF + stage * (L::K_BYTES + L::V_BYTES);
          const uint32_t v_dst = k_dst + L::K_BYTES;
          mbar_arrive_expect_tx(k_full(stage), L::K_BYTES);
#pragma unroll
          for (int c = 0; c < L::DCH; ++c)
            tma_load_3d(k_dst + c * SUBTILE_BYTES, &map_k, k_full(stage), kv_head * D + c * 64, j * BLOCK_N, item.batch);
          mbar_arrive_expect_tx(v_full(stage), L::V_BYTES);
#pragma unroll
          for (int c = 0; c < L::DCH; ++c)
            tma_load_3d(v_dst + c * SUBTILE_BYTES, &map_v, v_full(stage), kv_head * D + c * 64, j * BLOCK_N, item.batch);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(BLOCK_M, BLOCK_N);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(BLOCK_M, D, false, true);  // V is MN-major
      auto issue_qk = [&](int t, int stage) {  // S_t = Q_t · K^T with K in ring stage `stage`
        const uint32_t k_src = base + L::KV_OFF + stage * (L::K_BYTES + L::V_BYTES);
        const uint32_t acc = tmem_base + (uint32_t)(t * BLOCK_N);
#pragma unroll
        for (int c = 0; c < L::DCH; ++c) {
          const uint64_t desc_q = umma_desc_k_major_sw128(base + L::Q_OFF + t * L::Q_BYTES + c * SUBTILE_BYTES);
          const uint64_t desc_k = umma_desc_k_major_sw128(k_src + c * SUBTILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ss(acc, umma_desc_advance_k(desc_q, kk * 32), umma_desc_advance_k(desc_k, kk * 32), idesc_qk,
                         (c | kk) != 0 ? 1u : 0u);
        }
        umma_commit(s_ready(t));
      };
      // O_t (+)= P_t · V over keys [64*half, 64*half+64) of the block in ring stage `stage`; P_t is packed bf16 in the
      // first 64 columns of S_t; `first` = first block of the item (O_t is overwritten, not accumulated)
      auto issue_pv = [&](int t, int stage, int half, bool first) {
        const uint32_t v_src = base + L::KV_OFF + stage * (L::K_BYTES + L::V_BYTES) + L::K_BYTES;
        const uint64_t desc_v = umma_desc_mn_major_sw128(v_src, SUBTILE_BYTES);
        const uint32_t p_addr = tmem_base + (uint32_t)(t * BLOCK_N);
        const uint32_t o_addr = tmem_base + 256u + (uint32_t)(t * 128);
#pragma unroll
        for (int kk = half * 4; kk < half * 4 + 4; ++kk)
          umma_bf16_ts(o_addr, p_addr + (uint32_t)(kk * 8), umma_desc_advance_k(desc_v, kk * 2048), idesc_pv,
                       (!first || kk != 0) ? 1u : 0u);
        if (half == 1) umma_commit(o_done(t));
      };
      bool ok = true;
      int kv_count = 0;               // key/value blocks consumed so far (ring stage and parity)
      int blocks_done[Q_TILES] = {};  // score blocks issued so far per tile (parity of s_ready / p_ready / o_done)
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!(ok = mbar_wait(item_full(slot), (uint32_t)(n >> 1) & 1u, abort_flag, status_word, kWaitItem))) break;
        const int index = item_slot[slot];
        if (index < 0) break;
        const Item item = decode(index);
        if (!(ok = mbar_wait(q_full, (uint32_t)n & 1u, abort_flag, status_word, kWaitQ))) break;
        if (!(ok = mbar_wait(k_full(kv_count & 1), (uint32_t)(kv_count >> 1) & 1u, abort_flag, status_word, kWaitK))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int t = 0; t < Q_TILES; ++t)
          if (0 < item.blocks_of[t]) issue_qk(t, kv_count & 1);
        for (int j = 0; ok && j < item.kv_blocks; ++j) {
          const int current = kv_count + j, next = current + 1;
          const int stage = current & 1;
          // every Q·K^T of the item has been issued once its last block is reached: Q may be refilled when they complete
          if (j == item.kv_blocks - 1) umma_commit(q_free);
          if (!(ok = mbar_wait(v_full(stage), (uint32_t)(current >> 1) & 1u, abort_flag, status_word, kWaitV))) break;
          bool next_k_ready = false;
#pragma unroll
          for (int t = 0; t < Q_TILES; ++t) {
            if (j < item.blocks_of[t]) {
              const uint32_t parity = (uint32_t)(blocks_done[t] + j) & 1u;
              if (j == 0 && n > 0) {
                // O_t is about to be overwritten: the previous item's epilogue must have read it
                if (!(ok = mbar_wait(o_free(t), (uint32_t)(n - 1) & 1u, abort_flag, status_word, kWaitOFree))) break;
              }
              // the first 64 keys of P arrive while the softmax warps still work on the last 64
              if (!(ok = mbar_wait(p_ready(t, 0), parity, abort_flag, status_word, kWaitPReady))) break;
              tcgen05_fence_after();
              issue_pv(t, stage, 0, j == 0);
              if (!(ok = mbar_wait(p_ready(t, 1), parity, abort_flag, status_word, kWaitPReady))) break;
              tcgen05_fence_after();
              issue_pv(t, stage, 1, j == 0);
            }
            if (j + 1 < item.blocks_of[t]) {
              if (!next_k_ready) {
                if (!(ok = mbar_wait(k_full(next & 1), (uint32_t)(next >> 1) & 1u, abort_flag, status_word, kWaitK))) break;
                tcgen05_fence_after();
                next_k_ready = true;
              }
              issue_qk(t, next & 1);  // overwrites S_t/P_t: ordered after PV_t(j) on the tensor pipe
            }
          }
          if (ok) umma_commit(kv_empty(stage));
        }
        kv_count += item.kv_blocks;
#pragma unroll
        for (int t = 0; t < Q_TILES; ++t) blocks_done[t] += item.blocks_of[t];
        if (ok) mbar_arrive(item_empty(slot));
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ---------------- softmax + epilogue: warps 4..7 own tile 0, warps 8..11 own tile 1 ----------------
    const int tile = (warp - 4) >> 2;
    const int quadrant = warp & 3;          // TMEM lanes [32*quadrant, +32) are the ones this warp may touch
    const int row = quadrant * 32 + lane;   // row of the query tile == TMEM lane
    const uint32_t lane_base = (uint32_t)(quadrant * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + (uint32_t)(tile * BLOCK_N);
    const uint32_t o_addr = tmem_base + lane_base + 256u + (uint32_t)(tile * 128);
    bool ok = true;
    int blocks_done = 0;  // score blocks of this tile consumed so far, over all items (barrier parities)
    for (int n = 0; ok; ++n) {
    const int slot = n & 1;
    ok = mbar_wait(item_full(slot), (uint32_t)(n >> 1) & 1u, abort_flag, status_word, kWaitItem);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const int index = item_slot[slot];
    if (index < 0) break;
    const Item item = decode(index);
    const int pair = item.pair, head = item.head, batch = item.batch;
    const int q0 = (pair * Q_TILES + tile) * BLOCK_M;
    const int query = q0 + row;
    const int my_blocks = tile == 0 ? item.blocks_of[0] : item.blocks_of[1];
    float used_max = -INFINITY;             // running maximum (scaled, log2 units) the exponentials refer to
    float row_sum = 0.0f;
    for (int j = 0; j < my_blocks; ++j) {
      ok = mbar_wait(s_ready(tile), (uint32_t)(blocks_done + j) & 1u, abort_flag, status_word, kWaitSReady);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      uint32_t s[BLOCK_N];
#pragma unroll
      for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk)
        tmem_ld_32x32b_x32(s_addr + (uint32_t)(chunk * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[chunk * 32]));
      tmem_ld_wait();
      const int key0 = j * BLOCK_N;
      // only blocks that cross the causal diagonal or the end of the sequence need masking
      if ((CAUSAL && key0 + BLOCK_N - 1 > q0) || (key0 + BLOCK_N > seq)) {
        const int key_limit = (CAUSAL ? min(query, seq - 1) : seq - 1) - key0;  // largest visible column
#pragma unroll
        for (int i = 0; i < BLOCK_N; ++i)
          if (i > key_limit) s[i] = 0xff800000u;  // -inf
      }
      // four independent chains instead of one 128-long dependency chain
      float max0 = -INFINITY, max1 = -INFINITY, max2 = -INFINITY, max3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BLOCK_N; i += 8) {
        max0 = fmax3(max0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        max1 = fmax3(max1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        max2 = fmax3(max2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        max3 = fmax3(max3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      const float block_max = fmaxf(fmaxf(max0, max1), fmaxf(max2, max3));
      const float candidate = fmaxf(used_max, block_max * scale_log2e);  // scale > 0 commutes with max
      // O stays in TMEM; it is rescaled only when some row of this warp outgrows the threshold
      const bool grow = candidate > used_max + RESCALE_THRESHOLD;        // also true on the first finite block
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = candidate == -INFINITY ? 1.0f : fast_exp2(used_max - candidate);  // used_max = -inf gives 0
        row_sum *= alpha;
        used_max = candidate;
        if (j > 0) {
          // P·V of the previous block must have landed in O before it is rescaled
          ok = mbar_wait(o_done(tile), (uint32_t)(blocks_done + j - 1) & 1u, abort_flag, status_word, kWaitODone);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tcgen05_fence_after();
#pragma unroll
          for (int chunk = 0; chunk < D / 32; ++chunk) {
            uint32_t acc[32];
            tmem_ld_32x32b_x32(o_addr + (uint32_t)(chunk * 32), acc);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
            tmem_st_32x32b_x32(o_addr + (uint32_t)(chunk * 32), acc);
          }
        }
      }
      const float shift = used_max == -INFINITY ? 0.0f : -used_max;  // fully masked so far: 2^(-inf) = 0
      float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
      // Two halves of 64 keys; each is published as soon as it is in TMEM so P·V starts on the first
      // half while the second is still being exponentiated.  Packed in place: word i/2 of `s` is free
      // once scores i and i+1 have been consumed.  P overwrites the first 64 columns of this tile's S
      // (each thread only touches its own lane).
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int i = half * 64; i < half * 64 + 64; i += 4) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), scale_log2e, shift));
          const float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), scale_log2e, shift));
          const float p2 = fast_exp2(fmaf(__uint_as_float(s[i + 2]), scale_log2e, shift));
          const float p3 = fast_exp2(fmaf(__uint_as_float(s[i + 3]), scale_log2e, shift));
          sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
          const __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1);  // low half = even key
          const __nv_bfloat162 hi = __floats2bfloat162_rn(p2, p3);
          s[i >> 1] = *reinterpret_cast<const uint32_t*>(&lo);
          s[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&hi);
          if (half == 1 && i == 64 + DEFER_KEYS - 4) {
            // the first half's store has had DEFER_KEYS exponentials of time to land: publish it now
            tmem_st_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready(tile, 0));
          }
        }
        tmem_st_32x32b_x32(s_addr + (uint32_t)(half * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[half * 32]));
        if (half == 1) {
          tmem_st_wait();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_ready(tile, 1));
        }
      }
      row_sum += (sum0 + sum1) + (sum2 + sum3);
    }
    if (ok && my_blocks > 0) {
      ok = mbar_wait(o_done(tile), (uint32_t)(blocks_done + my_blocks - 1) & 1u, abort_flag, status_word, kWaitODone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && my_blocks > 0) {
      tcgen05_fence_after();
      const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
      const size_t out_batch = (size_t)(dst.batch_offset + batch);
      if constexpr (!GATHER) {
        __nv_bfloat16* row_out = static_cast<__nv_bfloat16*>(dst.out[0]) + ((out_batch * seq + query) * heads + head) * D;
#pragma unroll
        for (int chunk = 0; chunk < D / 32; ++chunk) {
          uint32_t acc[32];
          tmem_ld_32x32b_x32(o_addr + (uint32_t)(chunk * 32), acc);
          tmem_ld_wait();
          if (query < seq) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t word[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 pair2 = __floats2bfloat162_rn(__uint_as_float(acc[v * 8 + 2 * i]) * inv,
                                                                   __uint_as_float(acc[v * 8 + 2 * i + 1]) * inv);
                word[i] = *reinterpret_cast<const uint32_t*>(&pair2);
              }
              *reinterpret_cast<uint4*>(row_out + chunk * 32 + v * 8) = make_uint4(word[0], word[1], word[2], word[3]);
            }
          }
        }
      } else {
        // stage this warp's 32 rows in its quarter of the tile's Q buffer (all Q·K^T of this tile are complete);
        // 16-byte pieces are XOR-swizzled by row so that neither the row-wise writes nor the piece-wise reads conflict
        constexpr int ROW_BYTES = D * 2, PIECES = ROW_BYTES / 16;
        uint8_t* stage = aligned + L::Q_OFF + tile * L::Q_BYTES + quadrant * 32 * ROW_BYTES;
#pragma unroll
        for (int chunk = 0; chunk < D / 32; ++chunk) {
          uint32_t acc[32];
          tmem_ld_32x32b_x32(o_addr + (uint32_t)(chunk * 32), acc);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t word[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __nv_bfloat162 pair2 = __floats2bfloat162_rn(__uint_as_float(acc[v * 8 + 2 * i]) * inv,
                                                                 __uint_as_float(acc[v * 8 + 2 * i + 1]) * inv);
              word[i] = *reinterpret_cast<const uint32_t*>(&pair2);
            }
            const int piece = chunk * 4 + v;
            *reinterpret_cast<uint4*>(stage + lane * ROW_BYTES + ((piece ^ (lane & (PIECES - 1))) * 16)) =
                make_uint4(word[0], word[1], word[2], word[3]);
          }
        }
        __syncwarp();
        constexpr int ROWS_PER_STEP = 32 / PIECES;
        const int piece = lane % PIECES;
#pragma unroll
        for (int step = 0; step < PIECES; ++step) {
          const int r = step * ROWS_PER_STEP + lane / PIECES;
          const uint4 value = *reinterpret_cast<const uint4*>(stage + r * ROW_BYTES + ((piece ^ (r & (PIECES - 1))) * 16));
          const int row_query = q0 + quadrant * 32 + r;
          if (row_query < seq) {
            const size_t offset = (((out_batch * seq + row_query) * heads + head) * D) * 2 + (size_t)piece * 16;
            for (int d = 0; d < dst.count; ++d) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst.out[d]) + offset) = value;
          }
        }
      }
      // natural-log sum of exponentials of the scaled scores
      if (query < seq) {
        const float value = row_sum > 0.0f ? (used_max + log2f(row_sum)) * 0.6931471805599453f : -INFINITY;
        const size_t offset = (out_batch * heads + head) * seq + query;
        if constexpr (GATHER) {
          for (int d = 0; d < dst.count; ++d) dst.lse[d][offset] = value;
        } else {
          dst.lse[0][offset] = value;
        }
      }
    }
    if (!ok) break;
    // this item is finished for the warp: O_t may be overwritten, the ring slot (and, in the gather form, the
    // staging rows in Q) reused
    tcgen05_fence_before();
    if constexpr (GATHER) fence_proxy_async();  // the staged rows were read through the generic proxy; TMA refills them
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(o_free(tile));
      if constexpr (GATHER) mbar_arrive(q_free);
      mbar_arrive(item_empty(slot));
    }
    blocks_done += my_blocks;
    }  // items
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // a wait was abandoned: give copies that may still be in flight a bounded time to land
    const unsigned long long started = global_timer_ns();
    while (global_timer_ns() - started < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ---- plain SIMT kernel for head dims the tensor-core kernel does not cover -------------------------
// One CTA per (query, head, batch); scores live in shared memory (seq <= 8192).
__global__ void attn_fwd_generic_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                        const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out,
                                        float* __restrict__ lse, int seq, int heads, int kv_heads, int dim, int causal,
                                        float scale) {
  extern __shared__ float scores[];
  __shared__ float reduce[32];
  const int query = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (heads / kv_heads);
  const int last_key = causal ? query : seq - 1;
  const __nv_bfloat16* q_row = q + (((size_t)batch * seq + query) * heads + head) * dim;
  float local_max = -INFINITY;
  for (int key = threadIdx.x; key <= last_key; key += blockDim.x) {
    const __nv_bfloat16* k_row = k + (((size_t)batch * seq + key) * kv_heads + kv_head) * dim;
    float acc = 0.0f;
    for (int d = 0; d < dim; ++d) acc = fmaf(__bfloat162float(q_row[d]), __bfloat162float(k_row[d]), acc);
    acc *= scale;
    scores[key] = acc;
    local_max = fmaxf(local_max, acc);
  }
  auto block_reduce = [&](float value, bool is_max) {
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, value, offset);
      value = is_max ? fmaxf(value, other) : value + other;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) reduce[threadIdx.x >> 5] = value;
    __syncthreads();
    float total = is_max ? -INFINITY : 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total = is_max ? fmaxf(total, reduce[w]) : total + reduce[w];
    return total;
  };
  const float row_max = block_reduce(local_max, true);
  float local_sum = 0.0f;
  for (int key = threadIdx.x; key <= last_key; key += blockDim.x) {
    const float p = expf(scores[key] - row_max);
    scores[key] = p;
    local_sum += p;
  }
  const float row_sum = block_reduce(local_sum, false);
  __syncthreads();
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float acc = 0.0f;
    for (int key = 0; key <= last_key; ++key)
      acc = fmaf(scores[key], __bfloat162float(v[(((size_t)batch * seq + key) * kv_heads + kv_head) * dim + d]), acc);
    out[(((size_t)batch * seq + query) * heads + head) * dim + d] = __float2bfloat16_rn(acc / row_sum);
  }
  if (threadIdx.x == 0) lse[((size_t)batch * heads + head) * seq + query] = logf(row_sum) + row_max;
}

constexpr int kMaxDevices = 64;

// Work counters of the persistent kernel: a small pool handed out round-robin, so launches in flight at the same
// time (different streams, recorded graphs) do not share one unless more than kWorkCounters of them overlap.
constexpr int kWorkCounters = 256;
__device__ int g_attention_work_counters[kWorkCounters];

int* next_work_counter() {
  static std::atomic<unsigned> next{0};
  int* base = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_attention_work_counters) != cudaSuccess || !base) return nullptr;
  return base + (next.fetch_add(1) % kWorkCounters);
}

template <int D, bool CAUSAL, bool GATHER>
int launch_tensor_to(const void* q, const void* k, const void* v, const OutputDestinations& dst, int batch, int seq, int heads,
                     int kv_heads, cudaStream_t stream) {
  alignas(64) CUtensorMap map_q, map_k, map_v;
  if (int status = encode_tensormap_3d(&map_q, BB200_BF16, q, (uint64_t)heads * D, (uint64_t)seq, (uint64_t)batch,
                                       (uint64_t)heads * D * 2, (uint64_t)seq * heads * D * 2, 64, BLOCK_M, 1, 3))
    return status;
  if (int status = encode_tensormap_3d(&map_k, BB200_BF16, k, (uint64_t)kv_heads * D, (uint64_t)seq, (uint64_t)batch,
                                       (uint64_t)kv_heads * D * 2, (uint64_t)seq * kv_heads * D * 2, 64, BLOCK_N, 1, 3))
    return status;
  if (int status = encode_tensormap_3d(&map_v, BB200_BF16, v, (uint64_t)kv_heads * D, (uint64_t)seq, (uint64_t)batch,
                                       (uint64_t)kv_heads * D * 2, (uint64_t)seq * kv_heads * D * 2, 64, BLOCK_N, 1, 3))
    return status;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(BB200_E_NO_DRIVER, "attention: no CUDA device is current");
  static std::atomic<bool> configured[kMaxDevices];  // setting the attribute twice from two threads is harmless
  if (!configured[device]) {
    if (int status = check_runtime(cudaFuncSetAttribute(attn_fwd_kernel<D, CAUSAL, GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        Smem<D>::TOTAL),
                                   "cudaFuncSetAttribute(attention smem)"))
      return status;
    configured[device] = true;
  }
  const float scale_log2e = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  const int q_blocks = (seq + BLOCK_M - 1) / BLOCK_M;
  const long long items = (long long)((q_blocks + Q_TILES - 1) / Q_TILES) * heads * batch;
  if (items > 0x7fffffff - 4096) return fail(BB200_E_UNSUPPORTED_SHAPE, "attention: too many query tiles");
  static std::atomic<int> sm_counts[kMaxDevices];
  int sm_count = sm_counts[device].load(std::memory_order_relaxed);
  if (sm_count == 0) {
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sm_count = 0;
    sm_counts[device].store(sm_count, std::memory_order_relaxed);
  }
  if (sm_count <= 0) return fail(BB200_E_NO_DRIVER, "attention: could not query the SM count");
  // the CTAs draw their work items from a counter that this launch zeroes first (on the same stream); launches that
  // may overlap on the GPU get different counters
  int* counter = next_work_counter();
  if (!counter) return fail(BB200_E_NO_DRIVER, "attention: the work counters have no device address");
  if (int status = check_runtime(cudaMemsetAsync(counter, 0, sizeof(int), stream), "cudaMemsetAsync(attention work counter)")) return status;
  const int grid = (int)(items < sm_count ? items : sm_count);
  attn_fwd_kernel<D, CAUSAL, GATHER><<<grid, THREADS, Smem<D>::TOTAL, stream>>>(
      map_q, map_k, map_v, dst, seq, heads, kv_heads, batch, scale_log2e, counter, device_status_word());
  return check_launch("attention kernel launch");
}

template <int D, bool CAUSAL>
int launch_tensor(const void* q, const void* k, const void* v, const OutputDestinations& dst, int batch, int seq, int heads,
                  int kv_heads, cudaStream_t stream) {
  if (dst.count == 1 && dst.batch_offset == 0)
    return launch_tensor_to<D, CAUSAL, false>(q, k, v, dst, batch, seq, heads, kv_heads, stream);
  return launch_tensor_to<D, CAUSAL, true>(q, k, v, dst, batch, seq, heads, kv_heads, stream);
}

}  // namespace
}  // namespace bb200

using namespace bb200;

static int attention_fwd_to(const void* q, const void* k, const void* v, const OutputDestinations& dst, int batch, int seq,
                            int heads, int kv_heads, int head_dim, int causal, void* stream) {
  if (!q || !k || !v) return fail(BB200_E_INVALID_ARGUMENT, "attention: null tensor pointer");
  if (batch <= 0 || seq <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0)
    return fail(BB200_E_INVALID_ARGUMENT, "attention: extents must be > 0");
  if (heads % kv_heads) return fail(BB200_E_INVALID_ARGUMENT, "attention: heads=%d must be divisible by kv_heads=%d", heads, kv_heads);
  if (batch > 65535 || heads > 65535) return fail(BB200_E_UNSUPPORTED_SHAPE, "attention: batch and heads are limited to 65535");
  bool outputs_aligned = true;
  for (int d = 0; d < dst.count; ++d) {
    if (!dst.out[d] || !dst.lse[d]) return fail(BB200_E_INVALID_ARGUMENT, "attention: null tensor pointer");
    outputs_aligned = outputs_aligned && aligned16(dst.out[d]);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tensor_path = (head_dim == 64 || head_dim == 128) && aligned16(q) && aligned16(k) && aligned16(v) && outputs_aligned;
  if (tensor_path) {
    if (head_dim == 128)
      return causal ? launch_tensor<128, true>(q, k, v, dst, batch, seq, heads, kv_heads, s)
                    : launch_tensor<128, false>(q, k, v, dst, batch, seq, heads, kv_heads, s);
    return causal ? launch_tensor<64, true>(q, k, v, dst, batch, seq, heads, kv_heads, s)
                  : launch_tensor<64, false>(q, k, v, dst, batch, seq, heads, kv_heads, s);
  }
  if (dst.count != 1 || dst.batch_offset != 0)
    return fail(BB200_E_UNSUPPORTED_SHAPE, "attention (gather): only head_dim 64 and 128 with 16-byte aligned tensors are supported");
  if (seq > 8192) return fail(BB200_E_UNSUPPORTED_SHAPE, "attention: head_dim=%d with seq=%d > 8192 is not supported", head_dim, seq);
  dim3 grid(seq, heads, batch);
  attn_fwd_generic_kernel<<<grid, 128, (size_t)seq * sizeof(float), s>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      static_cast<__nv_bfloat16*>(dst.out[0]), dst.lse[0], seq, heads, kv_heads, head_dim, causal, 1.0f / sqrtf((float)head_dim));
  return check_launch("attention (generic) kernel launch");
}

extern "C" int bb200_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int seq,
                                   int heads, int kv_heads, int head_dim, int causal, void* stream) {
  OutputDestinations single = {};
  single.out[0] = out;
  single.lse[0] = lse;
  single.count = 1;
  single.batch_offset = 0;
  return attention_fwd_to(q, k, v, single, batch, seq, heads, kv_heads, head_dim, causal, stream);
}

extern "C" int bb200_attention_fwd_gather(const void* q, const void* k, const void* v, void* const* out_destinations,
                                          float* const* lse_destinations, int destination_count, int batch_offset, int batch,
                                          int seq, int heads, int kv_heads, int head_dim, int causal, void* stream) {
  if (!out_destinations || !lse_destinations || destination_count < 1 || destination_count > kMaxDestinations)
    return fail(BB200_E_INVALID_ARGUMENT, "attention (gather): 1..%d destination buffers are needed (got %d)", kMaxDestinations,
                destination_count);
  if (batch_offset < 0) return fail(BB200_E_INVALID_ARGUMENT, "attention (gather): batch_offset must be >= 0");
  OutputDestinations all = {};
  for (int d = 0; d < destination_count; ++d) {
    all.out[d] = out_destinations[d];
    all.lse[d] = lse_destinations[d];
  }
  all.count = destination_count;
  all.batch_offset = batch_offset;
  return attention_fwd_to(q, k, v, all, batch, seq, heads, kv_heads, head_dim, causal, stream);
}

// attn_fwd_tcgen05.cu — softmax attention forward for sm_100a (bf16 in/out, fp32 online softmax).
//
//   out[b, q, h, :] = softmax_k( q·k / sqrt(D)  [masked to k <= q when causal] ) · v,   lse = ln Σ exp(...)
//
// Tensors are [batch, seq, heads, head_dim] row-major, so one (batch, head) slice is a matrix whose
// rows are `heads*head_dim` elements apart; TMA reads it through a 3-D map (head_dim*heads, seq,
// batch) and zero-fills rows past `seq`.
//
// One CTA handles one 128-query block of one (batch, head) and walks the key/value blocks of 128
// keys (only those at or below the diagonal when causal).  192 threads:
//   warp 0      TMA producer: Q once, then K and V blocks into a 2-stage shared-memory ring.
//   warp 1      MMA issuer (one elected thread):  S = Q·K^T  (tcgen05.mma, both operands K-major in
//               shared memory, fp32 S in TMEM, double buffered so the next block's S is computed
//               while this block's softmax runs), then  O_blk = P·V  (P from shared memory, V
//               consumed in place as an MN-major operand).
//   warps 2..5  softmax: thread = query row.  Two passes over S in TMEM (row max; then exp2, row sum
//               and P written as bf16 into 128-byte-swizzled shared memory), then the running
//               output is updated in registers:  o = o * 2^(m_old - m_new) + O_blk.
// Tensor-core bound (4·B·H·D·S(S+1)/2 flops causal); HBM traffic is ~4·B·S·H·D·2 bytes.
// Head dims other than 64/128 use a plain SIMT kernel below.
#include <cuda_bf16.h>
#include <math.h>

#include "bb200_internal.h"
#include "bb200_sm100.cuh"

namespace bb200 {
namespace {

using namespace sm100;

constexpr int BLOCK_M = 128, BLOCK_N = 128;
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr int SUBTILE_BYTES = 128 * 128;  // [128 rows, 64 bf16] with 128-byte rows

enum WaitCode { kWaitQ = 201, kWaitKvEmpty = 202, kWaitK = 203, kWaitV = 204, kWaitSFull = 205, kWaitSEmpty = 206,
                kWaitP = 207, kWaitO = 208 };

template <int D> struct Smem {
  static constexpr int DCH = D / 64;                       // 64-column sub-tiles per row block
  static constexpr int Q_BYTES = DCH * SUBTILE_BYTES;
  static constexpr int K_BYTES = DCH * SUBTILE_BYTES;
  static constexpr int V_BYTES = DCH * SUBTILE_BYTES;
  static constexpr int P_BYTES = 2 * SUBTILE_BYTES;        // [128 queries, 128 keys] bf16
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = Q_OFF + Q_BYTES;
  static constexpr int P_OFF = KV_OFF + KV_STAGES * (K_BYTES + V_BYTES);
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;       // barriers + alignment slack
};

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                int seq, int heads, int kv_heads, float scale_log2e, int* status_word) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_addr(smem_raw));
  const uint32_t bar_base = base + L::BAR_OFF;
  // barriers: q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, o_full
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (3 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (5 + s); };
  auto s_full = [&](int b) { return bar_base + 8u * (7 + b); };
  auto s_empty = [&](int b) { return bar_base + 8u * (9 + b); };
  const uint32_t p_full = bar_base + 8u * 11;
  const uint32_t o_full = bar_base + 8u * 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aligned + L::BAR_OFF + 8 * 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blocks = (seq + BLOCK_M - 1) / BLOCK_M;
  const int q_block = q_blocks - 1 - (int)blockIdx.x;  // longest causal rows first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (heads / kv_heads);
  const int q0 = q_block * BLOCK_M;
  const int kv_blocks_all = (seq + BLOCK_N - 1) / BLOCK_N;
  const int kv_blocks = CAUSAL ? min(q_block + 1, kv_blocks_all) : kv_blocks_all;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(s_empty(b), 128);
    }
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(smem_addr(tmem_slot), 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;          // two S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;    // O block: columns [256, 256+D)

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < L::DCH; ++c)
        tma_load_3d(base + L::Q_OFF + c * SUBTILE_BYTES, &map_q, q_full, head * D + c * 64, q0, batch);
      bool ok = true;
      for (int j = 0; ok && j < kv_blocks; ++j) {
        const int stage = j & 1;
        const uint32_t use_parity = (uint32_t)(j >> 1) & 1u;
        if (!(ok = mbar_wait(kv_empty(stage), use_parity ^ 1u, abort_flag, status_word, kWaitKvEmpty))) break;
        const uint32_t k_dst = base + L::KV_OFF + stage * (L::K_BYTES + L::V_BYTES);
        const uint32_t v_dst = k_dst + L::K_BYTES;
        mbar_arrive_expect_tx(k_full(stage), L::K_BYTES);
#pragma unroll
        for (int c = 0; c < L::DCH; ++c)
          tma_load_3d(k_dst + c * SUBTILE_BYTES, &map_k, k_full(stage), kv_head * D + c * 64, j * BLOCK_N, batch);
        mbar_arrive_expect_tx(v_full(stage), L::V_BYTES);
#pragma unroll
        for (int c = 0; c < L::DCH; ++c)
          tma_load_3d(v_dst + c * SUBTILE_BYTES, &map_v, v_full(stage), kv_head * D + c * 64, j * BLOCK_N, batch);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(BLOCK_M, BLOCK_N);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(BLOCK_M, D, false, true);  // V is MN-major
      auto issue_qk = [&](int j) {
        const int stage = j & 1;
        const uint32_t k_src = base + L::KV_OFF + stage * (L::K_BYTES + L::V_BYTES);
        const uint32_t acc = tmem_s + (uint32_t)((j & 1) * BLOCK_N);
#pragma unroll
        for (int c = 0; c < L::DCH; ++c) {
          const uint64_t desc_q = umma_desc_k_major_sw128(base + L::Q_OFF + c * SUBTILE_BYTES);
          const uint64_t desc_k = umma_desc_k_major_sw128(k_src + c * SUBTILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ss(acc, umma_desc_advance_k(desc_q, kk * 32), umma_desc_advance_k(desc_k, kk * 32), idesc_qk,
                         (c | kk) != 0 ? 1u : 0u);
        }
        umma_commit(s_full(j & 1));
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, status_word, kWaitQ);
      if (ok) ok = mbar_wait(k_full(0), 0, abort_flag, status_word, kWaitK);
      if (ok) {
        tcgen05_fence_after();
        issue_qk(0);
      }
      for (int j = 0; ok && j < kv_blocks; ++j) {
        const int stage = j & 1;
        const uint32_t use_parity = (uint32_t)(j >> 1) & 1u;
        if (j + 1 < kv_blocks) {
          // S for the next block goes into the other buffer while this block's softmax runs
          const int next = j + 1;
          const uint32_t next_parity = (uint32_t)(next >> 1) & 1u;
          if (!(ok = mbar_wait(k_full(next & 1), next_parity, abort_flag, status_word, kWaitK))) break;
          if (!(ok = mbar_wait(s_empty(next & 1), next_parity ^ 1u, abort_flag, status_word, kWaitSEmpty))) break;
          tcgen05_fence_after();
          issue_qk(next);
        }
        if (!(ok = mbar_wait(p_full, (uint32_t)j & 1u, abort_flag, status_word, kWaitP))) break;
        if (!(ok = mbar_wait(v_full(stage), use_parity, abort_flag, status_word, kWaitV))) break;
        tcgen05_fence_after();
        const uint32_t v_src = base + L::KV_OFF + stage * (L::K_BYTES + L::V_BYTES) + L::K_BYTES;
        const uint64_t desc_v = umma_desc_mn_major_sw128(v_src, SUBTILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          const uint64_t desc_p = umma_desc_k_major_sw128(base + L::P_OFF + (kk >> 2) * SUBTILE_BYTES);
          umma_bf16_ss(tmem_o, umma_desc_advance_k(desc_p, (kk & 3) * 32), umma_desc_advance_k(desc_v, kk * 2048), idesc_pv,
                       kk != 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(kv_empty(stage));
      }
    }
  } else {
    // ---------------- softmax and output accumulation (warps 2..5) ----------------
    const int quadrant = warp & 3;
    const int row = quadrant * 32 + lane;   // row of the query block == TMEM lane
    const int query = q0 + row;
    const uint32_t lane_base = (uint32_t)(quadrant * 32) << 16;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.0f;
    float row_max = -INFINITY, row_sum = 0.0f;
    bool ok = true;
    for (int j = 0; j < kv_blocks; ++j) {
      const int buffer = j & 1;
      const uint32_t use_parity = (uint32_t)(j >> 1) & 1u;
      ok = mbar_wait(s_full(buffer), use_parity, abort_flag, status_word, kWaitSFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t s_addr = tmem_s + lane_base + (uint32_t)(buffer * BLOCK_N);
      const int key0 = j * BLOCK_N;
      // a block needs masking when it crosses the causal diagonal or the end of the sequence
      const bool masked_block = (CAUSAL && key0 + BLOCK_N - 1 > q0) || (key0 + BLOCK_N > seq);
      const int key_limit = CAUSAL ? min(query, seq - 1) : seq - 1;  // largest key index this row may see
      // pass 1: row maximum of the scaled scores
      float block_max = -INFINITY;
#pragma unroll 1
      for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(s_addr + (uint32_t)(chunk * 32), raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float t = __uint_as_float(raw[i]) * scale_log2e;
          if (masked_block && key0 + chunk * 32 + i > key_limit) t = -INFINITY;
          block_max = fmaxf(block_max, t);
        }
      }
      const float new_max = fmaxf(row_max, block_max);
      const float safe_max = new_max == -INFINITY ? 0.0f : new_max;  // fully masked so far: exp2(-inf - 0) = 0
      const float alpha = exp2f(row_max - safe_max);                 // row_max = -inf gives 0
      // pass 2: p = 2^(t - max), row sum, P as bf16 into swizzled shared memory
      float block_sum = 0.0f;
#pragma unroll 1
      for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(s_addr + (uint32_t)(chunk * 32), raw);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float t0 = __uint_as_float(raw[i]) * scale_log2e, t1 = __uint_as_float(raw[i + 1]) * scale_log2e;
          if (masked_block) {
            if (key0 + chunk * 32 + i > key_limit) t0 = -INFINITY;
            if (key0 + chunk * 32 + i + 1 > key_limit) t1 = -INFINITY;
          }
          const float p0 = exp2f(t0 - safe_max), p1 = exp2f(t1 - safe_max);
          // the row sum uses the bf16-rounded probabilities that the P·V product will see
          const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
          block_sum += __low2float(pair) + __high2float(pair);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        // 32 keys = four 16-byte chunks of this row; chunk index is XOR-swizzled with (row % 8)
        const int sub = chunk >> 1;                      // which [128, 64] sub-tile of P
        const int first = (chunk & 1) * 4;               // first 16-byte chunk within the 128-byte row
        uint8_t* p_row = aligned + L::P_OFF + sub * SUBTILE_BYTES + row * 128;
#pragma unroll
        for (int v = 0; v < 4; ++v)
          *reinterpret_cast<uint4*>(p_row + (((first + v) ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
      }
      // S buffer fully read: hand it back; P written: publish it to the tensor core (async proxy)
      tcgen05_fence_before();
      mbar_arrive(s_empty(buffer));
      fence_proxy_async();
      mbar_arrive(p_full);
      row_sum = row_sum * alpha + block_sum;
      row_max = new_max;
      // O_blk = P·V, then o = o * alpha + O_blk
      ok = mbar_wait(o_full, (uint32_t)j & 1u, abort_flag, status_word, kWaitO);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
#pragma unroll
      for (int chunk = 0; chunk < D / 32; ++chunk) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(tmem_o + lane_base + (uint32_t)(chunk * 32), raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[chunk * 32 + i] = fmaf(o[chunk * 32 + i], alpha, __uint_as_float(raw[i]));
      }
      tcgen05_fence_before();
    }
    if (ok && query < seq) {
      const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
      __nv_bfloat16* dst = out + (((size_t)batch * seq + query) * heads + head) * D;
#pragma unroll
      for (int v = 0; v < D / 8; ++v) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 pair = __floats2bfloat162_rn(o[v * 8 + 2 * i] * inv, o[v * 8 + 2 * i + 1] * inv);
          packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      // natural-log sum of exponentials of the scaled scores
      lse[((size_t)batch * heads + head) * seq + query] =
          row_sum > 0.0f ? (row_max + log2f(row_sum)) * 0.6931471805599453f : -INFINITY;
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

template <int D, bool CAUSAL>
int launch_tensor(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int seq, int heads,
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
  static bool configured[kMaxDevices] = {};
  if (!configured[device]) {
    if (int status = check_runtime(cudaFuncSetAttribute(attn_fwd_kernel<D, CAUSAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        Smem<D>::TOTAL),
                                   "cudaFuncSetAttribute(attention smem)"))
      return status;
    configured[device] = true;
  }
  const float scale_log2e = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  dim3 grid((seq + BLOCK_M - 1) / BLOCK_M, heads, batch);
  attn_fwd_kernel<D, CAUSAL><<<grid, THREADS, Smem<D>::TOTAL, stream>>>(
      map_q, map_k, map_v, static_cast<__nv_bfloat16*>(out), lse, seq, heads, kv_heads, scale_log2e, device_status_word());
  return check_launch("attention kernel launch");
}

}  // namespace
}  // namespace bb200

using namespace bb200;

extern "C" int bb200_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int seq,
                                   int heads, int kv_heads, int head_dim, int causal, void* stream) {
  if (!q || !k || !v || !out || !lse) return fail(BB200_E_INVALID_ARGUMENT, "attention: null tensor pointer");
  if (batch <= 0 || seq <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0)
    return fail(BB200_E_INVALID_ARGUMENT, "attention: extents must be > 0");
  if (heads % kv_heads) return fail(BB200_E_INVALID_ARGUMENT, "attention: heads=%d must be divisible by kv_heads=%d", heads, kv_heads);
  if (batch > 65535 || heads > 65535) return fail(BB200_E_UNSUPPORTED_SHAPE, "attention: batch and heads are limited to 65535");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tensor_path = (head_dim == 64 || head_dim == 128) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out);
  if (tensor_path) {
    if (head_dim == 128)
      return causal ? launch_tensor<128, true>(q, k, v, out, lse, batch, seq, heads, kv_heads, s)
                    : launch_tensor<128, false>(q, k, v, out, lse, batch, seq, heads, kv_heads, s);
    return causal ? launch_tensor<64, true>(q, k, v, out, lse, batch, seq, heads, kv_heads, s)
                  : launch_tensor<64, false>(q, k, v, out, lse, batch, seq, heads, kv_heads, s);
  }
  if (seq > 8192) return fail(BB200_E_UNSUPPORTED_SHAPE, "attention: head_dim=%d with seq=%d > 8192 is not supported", head_dim, seq);
  dim3 grid(seq, heads, batch);
  attn_fwd_generic_kernel<<<grid, 128, (size_t)seq * sizeof(float), s>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      static_cast<__nv_bfloat16*>(out), lse, seq, heads, kv_heads, head_dim, causal, 1.0f / sqrtf((float)head_dim));
  return check_launch("attention (generic) kernel launch");
}

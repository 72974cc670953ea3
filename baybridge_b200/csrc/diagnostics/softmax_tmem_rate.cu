// softmax_tmem_rate.cu — stand-alone microbenchmark, not part of libbb200.so.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I.. -o softmax_tmem_rate softmax_tmem_rate.cu && ./softmax_tmem_rate
//
// Question: how fast is the attention kernel's softmax step by itself — the code of one score block exactly as the
// kernel runs it (128 fp32 scores of a row read from tensor memory, four max chains, the vote on the rescale, 128
// exponentials with scale-and-shift, four row-sum chains, bf16 packing in place, two 32-column stores back with the
// deferred wait) — with nothing else on the SM: no tensor-core work, no TMA, no barriers?  And how fast next to a
// tensor pipe kept busy by an independent stream of the kernel's two products (S = Q·K^T from shared memory, O += P·V
// with P from tensor memory) into other columns?  One CTA per SM, 4 or 8 softmax warps (one or two per scheduler);
// prints cycles per block per warp and per score per scheduler.
#include <cstdio>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../bb200_sm100.cuh"

using namespace bb200::sm100;

__device__ __forceinline__ float fast_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float fmax3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }

constexpr int BLOCK_N = 128, DEFER_KEYS = 32;
constexpr float RESCALE_THRESHOLD = 8.0f;

// VARIANT 0: the step as the kernel has it.  1: without the row maximum.  2: without the stores back to tensor memory.
// Warps 0..3: warp 0 issues the MMA stream (WITH_MMA), the others idle.  Warps 4..11 (or 4..7): softmax.
template <int VARIANT, bool WITH_MMA>
__global__ void __launch_bounds__(384, 1) kern(long long* clocks, float* sink, int* status, int blocks, int mma_groups, float scale_log2e) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_addr(smem_raw));
  for (int i = threadIdx.x; i < 64 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(aligned)[i] = 0;  // operands: zeros
  const uint32_t bar = base + 64 * 1024;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(aligned + 64 * 1024 + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) tmem_alloc(smem_addr(slot_ptr), 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t slot = *slot_ptr;
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");  // the register split of the kernel
    if (WITH_MMA && warp == 0 && elect_one()) {
      // columns [256, 384): a score accumulator (its first 64 columns double as the P operand); [384, 512): an O accumulator
      const uint64_t desc_a = umma_desc_k_major_sw128(base);
      const uint64_t desc_b = umma_desc_k_major_sw128(base + 16384);
      const uint64_t desc_v = umma_desc_mn_major_sw128(base + 16384, 16384);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(128, 128, false, true);
      constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(128, 128);
      for (int g = 0; g < mma_groups; ++g) {  // 16 MMAs = the tensor work of one 128-key block of one query tile
        for (int kk = 0; kk < 8; ++kk) umma_bf16_ts(slot + 384u, slot + 256u + (uint32_t)(kk * 8), umma_desc_advance_k(desc_v, kk * 2048), idesc_pv, 1);
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ss(slot + 256u, umma_desc_advance_k(desc_a, (kk & 3) * 32), umma_desc_advance_k(desc_b, (kk & 3) * 32), idesc_qk, kk != 0);
      }
      umma_commit(bar);
      mbar_wait(bar, 0, abort_flag, status, 900);
    }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
  const uint32_t s_addr = slot + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(((warp - 4) >> 2) * 128);
  {
    // scores like those of a real block: a few units around zero, different per lane and column
    uint32_t init[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int i = 0; i < 32; ++i) init[i] = __float_as_uint((float)(((threadIdx.x * 131 + (c * 32 + i) * 17) % 97) - 48) * 0.11f);
      tmem_st_32x32b_x32(s_addr + c * 32, init);
    }
    tmem_st_wait();
  }
  float used_max = -INFINITY, row_sum = 0.0f;
  const long long start = clock64();
  for (int j = 0; j < blocks; ++j) {
    const uint32_t block_addr = s_addr;
    uint32_t s[BLOCK_N];
#pragma unroll
    for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk)
      tmem_ld_32x32b_x32(block_addr + (uint32_t)(chunk * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[chunk * 32]));
    tmem_ld_wait();
    float block_max = __uint_as_float(s[0]) + 4.0f;
    if (VARIANT != 1) {
      float max0 = -INFINITY, max1 = -INFINITY, max2 = -INFINITY, max3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BLOCK_N; i += 8) {
        max0 = fmax3(max0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        max1 = fmax3(max1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        max2 = fmax3(max2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        max3 = fmax3(max3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      block_max = fmaxf(fmaxf(max0, max1), fmaxf(max2, max3));
    }
    const float candidate = fmaxf(used_max, block_max * scale_log2e);
    const bool grow = candidate > used_max + RESCALE_THRESHOLD;
    if (__any_sync(0xffffffffu, grow)) {
      const float alpha = candidate == -INFINITY ? 1.0f : fast_exp2(used_max - candidate);
      row_sum *= alpha;
      used_max = candidate;
    }
    const float shift = used_max == -INFINITY ? 0.0f : -used_max;
    float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int i = half * 64; i < half * 64 + 64; i += 4) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), scale_log2e, shift));
        const float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), scale_log2e, shift));
        const float p2 = fast_exp2(fmaf(__uint_as_float(s[i + 2]), scale_log2e, shift));
        const float p3 = fast_exp2(fmaf(__uint_as_float(s[i + 3]), scale_log2e, shift));
        sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
        const __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(p2, p3);
        s[i >> 1] = *reinterpret_cast<const uint32_t*>(&lo);
        s[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&hi);
        if (VARIANT != 2 && half == 1 && i == 64 + DEFER_KEYS - 4) {
          tmem_st_wait();
          tcgen05_fence_before();
          __syncwarp();
        }
      }
      if (VARIANT != 2) tmem_st_32x32b_x32(block_addr + (uint32_t)(half * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[half * 32]));
      if (VARIANT == 2) row_sum += __uint_as_float(s[half * 32 + 5]) * 1e-30f;
      if (VARIANT != 2 && half == 1) {
        tmem_st_wait();
        tcgen05_fence_before();
        __syncwarp();
      }
    }
    row_sum += (sum0 + sum1) + (sum2 + sum3);
    // put plausible scores back where P went, so the next visit of this buffer exponentiates sane numbers
    if (VARIANT != 2 && (j & 7) == 7) {
      uint32_t init[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) init[i] = __float_as_uint((float)(((threadIdx.x * 131 + i * 17 + j) % 97) - 48) * 0.11f);
      tmem_st_32x32b_x32(block_addr, init);
      tmem_st_32x32b_x32(block_addr + 32, init);
      tmem_st_wait();
    }
  }
  const long long end = clock64();
  sink[blockIdx.x * blockDim.x + threadIdx.x] = row_sum + used_max;
  if (threadIdx.x == 128 && blockIdx.x == 0) clocks[0] = end - start;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    tmem_dealloc(slot, 512);
  }
}

template <int VARIANT, bool WITH_MMA> void run(long long* clocks, float* sink, int* status, int softmax_warps) {
  const int blocks = 2000;
  const int threads = 128 + 32 * softmax_warps;
  const int smem = 64 * 1024 + 1024 + 256;
  cudaFuncSetAttribute(kern<VARIANT, WITH_MMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  // enough tensor work to cover the softmax run: 1024 cycles per group
  const int mma_groups = softmax_warps == 8 ? 5600 : 3600;
  for (int it = 0; it < 2; ++it) kern<VARIANT, WITH_MMA><<<148, threads, smem>>>(clocks, sink, status, blocks, mma_groups, 0.1275f);
  if (cudaDeviceSynchronize() != cudaSuccess) {
    printf("error: %s\n", cudaGetErrorString(cudaGetLastError()));
    return;
  }
  long long host = 0;
  cudaMemcpy(&host, clocks, 8, cudaMemcpyDeviceToHost);
  const double cycles = (double)host / blocks;
  static const char* const kVariants[] = {"as in the kernel", "without the row maximum", "without the stores"};
  printf("%-24s %s %d warps per scheduler : %8.1f cycles per block per warp, %6.2f cycles per score per scheduler\n", kVariants[VARIANT],
         WITH_MMA ? "tensor pipe busy," : "tensor pipe idle,", softmax_warps / 4, cycles, cycles / 128.0 / (softmax_warps / 4));
}

int main() {
  long long* clocks;
  float* sink;
  int* status;
  cudaMalloc(&clocks, 8);
  cudaMalloc(&sink, 148 * 384 * 4);
  cudaMalloc(&status, 4);
  cudaMemset(status, 0, 4);
  for (int softmax_warps : {4, 8}) {
    run<0, false>(clocks, sink, status, softmax_warps);
    run<1, false>(clocks, sink, status, softmax_warps);
    run<2, false>(clocks, sink, status, softmax_warps);
    run<0, true>(clocks, sink, status, softmax_warps);
    run<2, true>(clocks, sink, status, softmax_warps);
  }
  int host_status = 0;
  cudaMemcpy(&host_status, status, 4, cudaMemcpyDeviceToHost);
  printf("device status %d\n", host_status);
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}

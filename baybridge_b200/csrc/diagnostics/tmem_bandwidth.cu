// tmem_bandwidth.cu — stand-alone microbenchmark, not part of libbb200.so.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -I.. -o tmem_bandwidth tmem_bandwidth.cu && ./tmem_bandwidth
//
// Question: how many bytes per clock can the warps of one SM move between tensor memory and registers with
// `tcgen05.ld` / `tcgen05.st` (32x32b shapes, as the attention softmax uses them: a thread reads the 128 fp32 scores of
// its row, writes 64 words of packed probabilities back)?  One CTA per SM with 4 or 8 warps (one or two per lane
// quadrant); every warp repeats "read 128 columns of its 32 lanes" (MODE 0), "write 64 columns" (MODE 1) or both
// (MODE 2), with x16 / x32 / x64 instructions.  Prints cycles per repetition and bytes per clock per SM.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

#include "../bb200_sm100.cuh"

using namespace bb200::sm100;

template <int N> struct Regs { uint32_t r[N]; };

__device__ __forceinline__ void ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, "
      "%28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, "
      "%54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]),
        "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]),
        "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}

// MODE 0: loads, 1: stores, 2: both.  WIDTH: columns per instruction (16, 32 or 64).
template <int MODE, int WIDTH>
__global__ void __launch_bounds__(256, 1) kern(long long* clocks, uint32_t* sink, int reps) {
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) tmem_alloc(smem_addr(&slot), 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t base = slot + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((warp >> 2) * 256);  // the second warp of a quadrant takes other columns
  uint32_t keep = threadIdx.x;
  uint32_t packed[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) packed[i] = threadIdx.x * 64 + i;
  __syncthreads();
  const long long start = clock64();
  for (int r = 0; r < reps; ++r) {
    if (MODE == 0 || MODE == 2) {
      if constexpr (WIDTH == 64) {
        uint32_t s[128];
        ld64(base, *reinterpret_cast<uint32_t(*)[64]>(&s[0]));
        ld64(base + 64, *reinterpret_cast<uint32_t(*)[64]>(&s[64]));
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 128; i += 16) keep ^= s[i];
      } else if constexpr (WIDTH == 32) {
        uint32_t s[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 128; i += 16) keep ^= s[i];
      } else {
        uint32_t s[128];
#pragma unroll
        for (int c = 0; c < 8; ++c) tmem_ld_32x32b_x16(base + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&s[c * 16]));
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 128; i += 16) keep ^= s[i];
      }
    }
    if (MODE == 1 || MODE == 2) {
      packed[0] ^= keep;
      if constexpr (WIDTH >= 32) {
        tmem_st_32x32b_x32(base + 128, *reinterpret_cast<uint32_t(*)[32]>(&packed[0]));
        tmem_st_32x32b_x32(base + 160, *reinterpret_cast<uint32_t(*)[32]>(&packed[32]));
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_st_32x32b_x16(base + 128 + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&packed[c * 16]));
      }
      tmem_st_wait();
    }
  }
  const long long end = clock64();
  sink[blockIdx.x * blockDim.x + threadIdx.x] = keep ^ packed[5];
  if (threadIdx.x == 0 && blockIdx.x == 0) clocks[0] = end - start;
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    tmem_dealloc(slot, 512);
  }
}

template <int MODE, int WIDTH> void run(long long* clocks, uint32_t* sink, int threads) {
  const int reps = 4000;
  for (int it = 0; it < 2; ++it) kern<MODE, WIDTH><<<148, threads>>>(clocks, sink, reps);
  cudaDeviceSynchronize();
  long long host = 0;
  cudaMemcpy(&host, clocks, 8, cudaMemcpyDeviceToHost);
  const double cycles = (double)host / reps;
  const double bytes_per_warp = (MODE == 0 ? 128 : MODE == 1 ? 64 : 192) * 32 * 4.0;
  static const char* const kModes[] = {"read 128 columns", "write 64 columns", "read 128 + write 64"};
  printf("%-20s x%-2d  %d warps per SM : %8.1f cycles per repetition, %6.1f bytes per clock per SM\n", kModes[MODE], WIDTH, threads / 32, cycles,
         bytes_per_warp * (threads / 32) / cycles);
}

int main() {
  long long* clocks;
  uint32_t* sink;
  cudaMalloc(&clocks, 8);
  cudaMalloc(&sink, 148 * 256 * 4);
  for (int threads : {128, 256}) {
    run<0, 16>(clocks, sink, threads); run<0, 32>(clocks, sink, threads); run<0, 64>(clocks, sink, threads);
    run<1, 16>(clocks, sink, threads); run<1, 32>(clocks, sink, threads);
    run<2, 32>(clocks, sink, threads);
  }
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}

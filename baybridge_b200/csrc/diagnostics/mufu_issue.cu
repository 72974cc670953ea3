// mufu_issue.cu — stand-alone microbenchmark, not part of libbb200.so.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o mufu_issue mufu_issue.cu && ./mufu_issue
//
// Question: does an `ex2.approx` hold the warp scheduler's dispatch for its 8 cycles, or can FMA-pipe instructions
// issue underneath it?  Each element runs one ex2 (or a Cody-Waite cubic on the FMA pipe) plus one dependent fma and
// K independent filler instructions; the program prints cycles per element per warp for 1, 2 and 4 warps per
// scheduler.  FILL selects the filler: 0 `fma.rn.f32`, 1 `fma.rn.f32x2` (one packed instruction = two fmas), 2 `add.f32x2`,
// 3 three-input `max.f32` and 4 `cvt.rn.bf16x2.f32` (both on the ALU pipe).
// The attention kernel's softmax schedule was sized from these numbers.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ float fast_exp2(float x) { float y; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d; asm volatile("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d; asm volatile("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) { float d; asm volatile("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ unsigned pack_bf16x2(float a, float b) { unsigned d; asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a)); return d; }
template <int K, int MODE, int FILL>
__global__ void __launch_bounds__(512, 1) kern(const float* in, float* out, long long* clocks, int reps) {
  float v[32], acc[8];
  unsigned long long wide[8];
  unsigned packed[8];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = in[(threadIdx.x * 32 + i) & 1023];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    acc[i] = in[i] * 0.001f;
    wide[i] = ((unsigned long long)__float_as_uint(acc[i]) << 32) | __float_as_uint(acc[i] + 1.0f);
    packed[i] = 0;
  }
  const unsigned long long scale2 = ((unsigned long long)__float_as_uint(1.0001f) << 32) | __float_as_uint(1.0001f);
  const unsigned long long half2 = ((unsigned long long)__float_as_uint(0.5f) << 32) | __float_as_uint(0.5f);
  __syncthreads();
  const long long start = clock64();
  for (int r = 0; r < reps; ++r) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (MODE == 0) v[i] = fast_exp2(v[i]) * 0.0f + v[i];  // 1 ex2 + 1 ffma per element (dependent, but 32 independent chains)
      if (MODE == 2 && (i & 1) == 0) {  // one packed bf16x2 ex2 for elements i and i+1 (inputs packed first, result left packed)
        unsigned packed_in, packed_out;
        asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed_in) : "f"(v[i + 1]), "f"(v[i]));
        asm volatile("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(packed_out) : "r"(packed_in));
        v[i] = __uint_as_float(packed_out << 16) * 0.0f + v[i];
        v[i + 1] = __uint_as_float(packed_out & 0xffff0000u) * 0.0f + v[i + 1];
      }
      if (MODE == 3 && (i & 1) == 0) {  // the same with f16x2
        unsigned packed_in, packed_out;
        asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(packed_in) : "f"(v[i + 1]), "f"(v[i]));
        asm volatile("ex2.approx.f16x2 %0, %1;" : "=r"(packed_out) : "r"(packed_in));
        v[i] = __uint_as_float(packed_out << 16) * 0.0f + v[i];
        v[i + 1] = __uint_as_float(packed_out & 0xffff0000u) * 0.0f + v[i + 1];
      }
      if (MODE == 1) {  // scalar polynomial exp2: no MUFU
        float x = v[i];
        const float t = x + 12582912.0f;
        const float f = x - (t - 12582912.0f);
        float p = fmaf(0.05520550534129143f, f, 0.24261397123336792f);
        p = fmaf(p, f, 0.6932547688484192f);
        p = fmaf(p, f, 0.9999276995658875f);
        const float e = __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
        v[i] = e * 0.0f + v[i];
      }
#pragma unroll
      for (int k = 0; k < K; ++k) {  // independent filler
        const int a = (i + k) & 7;
        if (FILL == 0) acc[a] = fmaf(acc[a], 1.0001f, 0.5f);
        if (FILL == 1) wide[a] = fma2(wide[a], scale2, half2);
        if (FILL == 2) wide[a] = add2(wide[a], half2);
        if (FILL == 3) acc[a] = max3(acc[a], acc[(a + 1) & 7], acc[(a + 2) & 7]);
        if (FILL == 4) packed[a] ^= pack_bf16x2(acc[a], acc[(a + 1) & 7]);
      }
    }
  }
  const long long end = clock64();
  float s = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) s += v[i];
#pragma unroll
  for (int i = 0; i < 8; ++i) s += acc[i] + __uint_as_float((unsigned)(wide[i] >> 32)) + __uint_as_float((unsigned)wide[i]) + (float)packed[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
  if (threadIdx.x == 0 && blockIdx.x == 0) clocks[0] = end - start;
}
template <int K, int MODE, int FILL = 0> void run(const float* in, float* out, long long* clocks, int threads) {
  const int reps = 2000;
  for (int it = 0; it < 2; ++it) kern<K, MODE, FILL><<<148, threads>>>(in, out, clocks, reps);
  cudaDeviceSynchronize();
  long long host; cudaMemcpy(&host, clocks, 8, cudaMemcpyDeviceToHost);
  static const char* const kFillers[] = {"fma.f32", "fma.f32x2", "add.f32x2", "max3.f32", "cvt.bf16x2"};
  printf("mode %d (%s) filler %s per element %d  warps/scheduler %d : %6.2f clk per element per warp\n", MODE, MODE == 0 ? "ex2" : MODE == 1 ? "polynomial" : MODE == 2 ? "ex2.bf16x2" : "ex2.f16x2",
         kFillers[FILL], K, threads / 128, (double)host / reps / 32);
}
int main() {
  float* in; float* out; long long* clocks;
  cudaMalloc(&in, 1024 * 4); cudaMalloc(&out, 148 * 512 * 4); cudaMalloc(&clocks, 8);
  float host[1024]; for (int i = 0; i < 1024; ++i) host[i] = -(float)((i * 37) % 101) * 0.05f;
  cudaMemcpy(in, host, sizeof(host), cudaMemcpyHostToDevice);
  for (int threads : {128, 256, 512}) {
    run<0, 0>(in, out, clocks, threads); run<1, 0>(in, out, clocks, threads); run<2, 0>(in, out, clocks, threads); run<3, 0>(in, out, clocks, threads);
    run<4, 0>(in, out, clocks, threads); run<6, 0>(in, out, clocks, threads); run<8, 0>(in, out, clocks, threads);
    run<0, 1>(in, out, clocks, threads); run<3, 1>(in, out, clocks, threads);
    run<0, 2>(in, out, clocks, threads); run<2, 2>(in, out, clocks, threads); run<0, 3>(in, out, clocks, threads); run<2, 3>(in, out, clocks, threads);
    run<1, 0, 1>(in, out, clocks, threads); run<2, 0, 1>(in, out, clocks, threads); run<4, 0, 1>(in, out, clocks, threads);
    run<1, 0, 2>(in, out, clocks, threads); run<2, 0, 2>(in, out, clocks, threads); run<4, 0, 2>(in, out, clocks, threads);
    run<1, 0, 3>(in, out, clocks, threads); run<2, 0, 3>(in, out, clocks, threads); run<4, 0, 3>(in, out, clocks, threads);
    run<1, 0, 4>(in, out, clocks, threads); run<2, 0, 4>(in, out, clocks, threads); run<4, 0, 4>(in, out, clocks, threads);
  }
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}

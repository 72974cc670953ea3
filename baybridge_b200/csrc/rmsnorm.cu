// rmsnorm.cu — RMSNorm forward for sm_100a: out = x * rsqrt(mean(x^2) + eps) * gamma.
//
// HBM-bound: every element of x is read exactly once and every element of out written once
// (algorithmic bytes per row = 2 * hidden * sizeof(T); gamma is reused from L2/L1).  One CTA
// owns one row: each thread keeps its share of the row in registers as 16-byte vectors, the
// sum of squares is reduced in fp32 with warp shuffles plus one shared-memory hop, and the
// scaled row is written back with streaming 16-byte stores.  Rows longer than the register
// budget fall back to a second read of the row (served by L2).
#include "bb200_elementwise.cuh"
#include "bb200_internal.h"

namespace bb200 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

// Block-wide sum; every thread receives the total.  `scratch` holds one float per warp.
template <int THREADS> __device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  if constexpr (THREADS == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = lane < THREADS / 32 ? scratch[lane] : 0.0f;
  return warp_sum(total);
}

// Where the normalised rows go.  Ordinarily one [rows, hidden] tensor.  In the gather form this GPU's rows are a
// row block of a taller tensor that every GPU of the box holds a copy of: each output vector is stored into all
// `count` copies (its own and, through peer-mapped pointers, the others') at row `row_offset + row`, so the output
// all-gather rides along with the kernel.
constexpr int kMaxDestinations = 8;
struct RowDestinations {
  void* p[kMaxDestinations];
  int count;
  size_t row_offset;
};

// VPT = 16-byte vectors per thread held in registers.  CACHED=false re-reads x in the second pass.
// GATHER = false is the single-destination kernel: its store is one instruction with no loop around it.
template <typename T, int THREADS, int VPT, bool CACHED, bool GATHER>
__global__ void __launch_bounds__(THREADS)
rmsnorm_rows(const T* __restrict__ x, const T* __restrict__ gamma, const __grid_constant__ RowDestinations dst, size_t rows, int hidden,
             size_t gamma_row_stride, float epsilon) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float scratch[32];
  dependent_launch_prologue();
  const size_t row = blockIdx.x;
  if (row >= rows) return;
  const T* __restrict__ xr = x + row * (size_t)hidden;
  const T* __restrict__ gr = gamma + row * gamma_row_stride;
  const size_t out_offset = (dst.row_offset + row) * (size_t)hidden;
  const int nvec = hidden / VEC;

  Pack<T, VEC> held[CACHED ? VPT : 1];
  float sum = 0.0f;
  if constexpr (CACHED) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      if (v < nvec) held[j] = load_stream<T, VEC>(xr + (size_t)v * VEC);
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      if (v < nvec) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float f = Conv<float, T>::widen(held[j].v[e]);
          sum = fmaf(f, f, sum);
        }
      }
    }
  } else {
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      // default caching: the row is read again below and should stay in L2
      const Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(xr + (size_t)v * VEC);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float f = Conv<float, T>::widen(p.v[e]);
        sum = fmaf(f, f, sum);
      }
    }
  }
  const float total = block_sum<THREADS>(sum, scratch);
  const float inv_rms = 1.0f / sqrtf(total / (float)hidden + epsilon);

  auto emit = [&](int v, const Pack<T, VEC>& p) {
    const Pack<T, VEC> g = *reinterpret_cast<const Pack<T, VEC>*>(gr + (size_t)v * VEC);  // cached: shared by all rows
    Pack<T, VEC> o;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      o.v[e] = Conv<float, T>::narrow(Conv<float, T>::widen(p.v[e]) * inv_rms * Conv<float, T>::widen(g.v[e]));
    if constexpr (GATHER) {
      for (int d = 0; d < dst.count; ++d) store_stream<T, VEC>(static_cast<T*>(dst.p[d]) + out_offset + (size_t)v * VEC, o);
    } else {
      store_stream<T, VEC>(static_cast<T*>(dst.p[0]) + out_offset + (size_t)v * VEC, o);
    }
  };
  if constexpr (CACHED) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      if (v < nvec) emit(v, held[j]);
    }
  } else {
    for (int v = threadIdx.x; v < nvec; v += THREADS) emit(v, load_stream<T, VEC>(xr + (size_t)v * VEC));
  }
}

template <typename T, int THREADS, int VPT, bool CACHED>
int launch(const void* x, const void* gamma, const RowDestinations& out, size_t rows, size_t hidden, int gamma_is_full, float epsilon,
           cudaStream_t stream) {
  if (out.count == 1 && out.row_offset == 0)
    launch_dependent(rmsnorm_rows<T, THREADS, VPT, CACHED, false>, dim3((unsigned)rows), dim3(THREADS), 0, stream,
                     static_cast<const T*>(x), static_cast<const T*>(gamma), out, rows, (int)hidden,
                     (size_t)(gamma_is_full ? hidden : 0), epsilon);
  else
    rmsnorm_rows<T, THREADS, VPT, CACHED, true><<<(unsigned)rows, THREADS, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), out, rows, (int)hidden, gamma_is_full ? hidden : 0, epsilon);
  return check_launch("rmsnorm kernel launch");
}

template <typename T>
int dispatch(const void* x, const void* gamma, const RowDestinations& out, size_t rows, size_t hidden, int gamma_is_full, float epsilon,
             cudaStream_t stream) {
  constexpr size_t VEC = 16 / sizeof(T);
  if (hidden % VEC) return fail(BB200_E_UNSUPPORTED_SHAPE, "rmsnorm: hidden=%zu must be a multiple of %zu", hidden, VEC);
  const size_t nvec = hidden / VEC;
#define BB200_RMS(THREADS, VPT) \
  if (nvec <= (size_t)(THREADS) * (VPT)) return launch<T, THREADS, VPT, true>(x, gamma, out, rows, hidden, gamma_is_full, epsilon, stream)
  BB200_RMS(32, 1);
  BB200_RMS(64, 1);
  BB200_RMS(128, 1);
  BB200_RMS(128, 2);
  BB200_RMS(256, 2);
  BB200_RMS(256, 4);   // hidden 8192 bf16: 1024 vectors
  BB200_RMS(512, 4);
  BB200_RMS(1024, 4);
#undef BB200_RMS
  return launch<T, 1024, 1, false>(x, gamma, out, rows, hidden, gamma_is_full, epsilon, stream);
}

}  // namespace
}  // namespace bb200

using namespace bb200;

static int rmsnorm_into(bb200_dtype dtype, const void* x, const void* gamma, const RowDestinations& out, size_t rows, size_t hidden,
                        int gamma_is_full, float epsilon, void* stream) {
  if (!x || !gamma) return fail(BB200_E_INVALID_ARGUMENT, "rmsnorm: null tensor pointer");
  if (rows == 0 || hidden == 0) return fail(BB200_E_INVALID_ARGUMENT, "rmsnorm: rows and hidden must be > 0");
  if (rows > 0x7fffffffu) return fail(BB200_E_UNSUPPORTED_SHAPE, "rmsnorm: more than 2^31-1 rows");
  if (hidden > 0x7fffffffu) return fail(BB200_E_UNSUPPORTED_SHAPE, "rmsnorm: hidden exceeds 2^31-1");
  if (!aligned16(x) || !aligned16(gamma)) return fail(BB200_E_MISALIGNED, "rmsnorm: x, gamma and out must be 16-byte aligned");
  for (int d = 0; d < out.count; ++d) {
    if (!out.p[d]) return fail(BB200_E_INVALID_ARGUMENT, "rmsnorm: null tensor pointer");
    if (!aligned16(out.p[d])) return fail(BB200_E_MISALIGNED, "rmsnorm: x, gamma and out must be 16-byte aligned");
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BB200_BF16: return dispatch<__nv_bfloat16>(x, gamma, out, rows, hidden, gamma_is_full, epsilon, s);
    case BB200_F16: return dispatch<__half>(x, gamma, out, rows, hidden, gamma_is_full, epsilon, s);
    case BB200_F32: return dispatch<float>(x, gamma, out, rows, hidden, gamma_is_full, epsilon, s);
    default: return fail(BB200_E_INVALID_ARGUMENT, "rmsnorm: dtype %d is not bf16/f16/f32", (int)dtype);
  }
}

extern "C" int bb200_rmsnorm(bb200_dtype dtype, const void* x, const void* gamma, void* out, size_t rows, size_t hidden,
                             int gamma_is_full, float epsilon, void* stream) {
  RowDestinations single = {};
  single.p[0] = out;
  single.count = 1;
  single.row_offset = 0;
  return rmsnorm_into(dtype, x, gamma, single, rows, hidden, gamma_is_full, epsilon, stream);
}

extern "C" int bb200_rmsnorm_gather(bb200_dtype dtype, const void* x, const void* gamma, void* const* out_destinations,
                                    int destination_count, size_t row_offset, size_t rows, size_t hidden, int gamma_is_full,
                                    float epsilon, void* stream) {
  if (!out_destinations || destination_count < 1 || destination_count > kMaxDestinations)
    return fail(BB200_E_INVALID_ARGUMENT, "rmsnorm (gather): 1..%d destination buffers are needed (got %d)", kMaxDestinations, destination_count);
  RowDestinations all = {};
  for (int d = 0; d < destination_count; ++d) all.p[d] = out_destinations[d];
  all.count = destination_count;
  all.row_offset = row_offset;
  return rmsnorm_into(dtype, x, gamma, all, rows, hidden, gamma_is_full, epsilon, stream);
}

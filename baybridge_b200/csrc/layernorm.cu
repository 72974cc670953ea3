// layernorm.cu — LayerNorm forward with fused residual add for sm_100a:
//   mixed = x + residual;  out_resid = mixed;  out = (mixed - mean(mixed)) / sqrt(var(mixed) + eps) * weight + bias
//
// HBM-bound: x and residual are read once, out and out_resid written once (algorithmic bytes per row
// = 4 * hidden * sizeof(T); weight and bias are reused from cache).  One CTA owns one row; the mixed
// row stays in registers as fp32-convertible 16-byte vectors, mean and the centred sum of squares are
// reduced in fp32 (two block reductions), each output is rounded once.
#include "bb200_elementwise.cuh"
#include "bb200_internal.h"

namespace bb200 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

template <int THREADS> __device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  if constexpr (THREADS == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = lane < THREADS / 32 ? scratch[lane] : 0.0f;
  return warp_sum(total);
}

// Where the two outputs go.  Ordinarily one pair of tensors.  In the gather form this GPU's rows are the block starting at
// `row_offset` of taller tensors of which every GPU of the box holds a copy: each output vector is stored into all
// `count` copies (its own and, through peer-mapped pointers, the others').
constexpr int kMaxDestinations = 8;
struct LayerNormDestinations {
  void* out[kMaxDestinations];
  void* out_resid[kMaxDestinations];
  int count;
  size_t row_offset;
};

// GATHER = false keeps one unconditional store per output vector (a loop over destinations there costs bandwidth).
template <typename T, int THREADS, int VPT, bool GATHER>
__global__ void __launch_bounds__(THREADS)
layernorm_rows(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight, const T* __restrict__ bias,
               const __grid_constant__ LayerNormDestinations dst, size_t rows, int hidden, size_t weight_row_stride,
               size_t bias_row_stride, float epsilon) {
  constexpr int VEC = 16 / sizeof(T);
  T* __restrict__ out = static_cast<T*>(dst.out[0]);
  T* __restrict__ out_resid = static_cast<T*>(dst.out_resid[0]);
  __shared__ float scratch[32];
  dependent_launch_prologue();
  const size_t row = blockIdx.x;
  if (row >= rows) return;
  const size_t offset = row * (size_t)hidden;
  const size_t out_offset = (row + dst.row_offset) * (size_t)hidden;
  const int nvec = hidden / VEC;
  float mixed[VPT][VEC];
  float sum = 0.0f;
  {
    // every load of the row is issued before the first store: the stores cannot move above them
    Pack<T, VEC> a[VPT], b[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      if (v < nvec) {
        a[j] = load_stream<T, VEC>(x + offset + (size_t)v * VEC);
        b[j] = load_stream<T, VEC>(residual + offset + (size_t)v * VEC);
      }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      if (v < nvec) {
        Pack<T, VEC> r;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          mixed[j][e] = Conv<float, T>::widen(a[j].v[e]) + Conv<float, T>::widen(b[j].v[e]);
          sum += mixed[j][e];
          r.v[e] = Conv<float, T>::narrow(mixed[j][e]);
        }
        if constexpr (GATHER) {
          for (int d = 0; d < dst.count; ++d) store_stream<T, VEC>(static_cast<T*>(dst.out_resid[d]) + out_offset + (size_t)v * VEC, r);
        } else {
          store_stream<T, VEC>(out_resid + out_offset + (size_t)v * VEC, r);
        }
      }
    }
  }
  const float mean = block_sum<THREADS>(sum, scratch) / (float)hidden;
  float centred = 0.0f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
    if (v < nvec) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float d = mixed[j][e] - mean;
        centred = fmaf(d, d, centred);
      }
    }
  }
  const float inv_std = 1.0f / sqrtf(block_sum<THREADS>(centred, scratch) / (float)hidden + epsilon);
  const T* __restrict__ w_row = weight + row * weight_row_stride;
  const T* __restrict__ b_row = bias + row * bias_row_stride;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
    if (v < nvec) {
      const Pack<T, VEC> w = *reinterpret_cast<const Pack<T, VEC>*>(w_row + (size_t)v * VEC);
      const Pack<T, VEC> b = *reinterpret_cast<const Pack<T, VEC>*>(b_row + (size_t)v * VEC);
      Pack<T, VEC> o;
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        o.v[e] = Conv<float, T>::narrow((mixed[j][e] - mean) * inv_std * Conv<float, T>::widen(w.v[e]) + Conv<float, T>::widen(b.v[e]));
      if constexpr (GATHER) {
        for (int d = 0; d < dst.count; ++d) store_stream<T, VEC>(static_cast<T*>(dst.out[d]) + out_offset + (size_t)v * VEC, o);
      } else {
        store_stream<T, VEC>(out + out_offset + (size_t)v * VEC, o);
      }
    }
  }
}

template <typename T, int THREADS, int VPT>
int launch(const void* x, const void* residual, const void* weight, const void* bias, const LayerNormDestinations& dst, size_t rows,
           size_t hidden, int weight_is_full, int bias_is_full, float epsilon, cudaStream_t stream) {
  if (dst.count == 1 && dst.row_offset == 0) {
    launch_dependent(layernorm_rows<T, THREADS, VPT, false>, dim3((unsigned)rows), dim3(THREADS), 0, stream,
                     static_cast<const T*>(x), static_cast<const T*>(residual), static_cast<const T*>(weight),
                     static_cast<const T*>(bias), dst, rows, (int)hidden, (size_t)(weight_is_full ? hidden : 0),
                     (size_t)(bias_is_full ? hidden : 0), epsilon);
  } else {
    layernorm_rows<T, THREADS, VPT, true><<<(unsigned)rows, THREADS, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(residual), static_cast<const T*>(weight), static_cast<const T*>(bias), dst,
        rows, (int)hidden, weight_is_full ? hidden : 0, bias_is_full ? hidden : 0, epsilon);
  }
  return check_launch("layernorm kernel launch");
}

template <typename T>
int dispatch(const void* x, const void* residual, const void* weight, const void* bias, const LayerNormDestinations& dst, size_t rows,
             size_t hidden, int weight_is_full, int bias_is_full, float epsilon, cudaStream_t stream) {
  constexpr size_t VEC = 16 / sizeof(T);
  if (hidden % VEC) return fail(BB200_E_UNSUPPORTED_SHAPE, "layernorm: hidden=%zu must be a multiple of %zu", hidden, VEC);
  const size_t nvec = hidden / VEC;
#define BB200_LN(THREADS, VPT) \
  if (nvec <= (size_t)(THREADS) * (VPT)) \
    return launch<T, THREADS, VPT>(x, residual, weight, bias, dst, rows, hidden, weight_is_full, bias_is_full, epsilon, stream)
  BB200_LN(32, 1);
  BB200_LN(64, 1);
  BB200_LN(128, 1);
  BB200_LN(256, 1);
  BB200_LN(256, 2);
  BB200_LN(512, 2);   // hidden 8192 bf16: 1024 vectors
  BB200_LN(1024, 2);
  BB200_LN(1024, 4);
#undef BB200_LN
  return fail(BB200_E_UNSUPPORTED_SHAPE, "layernorm: hidden=%zu exceeds the %zu elements one CTA keeps in registers", hidden,
              (size_t)1024 * 4 * VEC);
}

}  // namespace
}  // namespace bb200

using namespace bb200;

static int layernorm_into(bb200_dtype dtype, const void* x, const void* residual, const void* weight, const void* bias,
                          const LayerNormDestinations& dst, size_t rows, size_t hidden, int weight_is_full, int bias_is_full,
                          float epsilon, void* stream) {
  if (!x || !residual || !weight || !bias) return fail(BB200_E_INVALID_ARGUMENT, "layernorm: null tensor pointer");
  if (rows == 0 || hidden == 0) return fail(BB200_E_INVALID_ARGUMENT, "layernorm: rows and hidden must be > 0");
  if (rows > 0x7fffffffu || hidden > 0x7fffffffu) return fail(BB200_E_UNSUPPORTED_SHAPE, "layernorm: extent exceeds 2^31-1");
  for (const void* p : {x, residual, weight, bias})
    if (!aligned16(p)) return fail(BB200_E_MISALIGNED, "layernorm: all tensors must be 16-byte aligned");
  for (int d = 0; d < dst.count; ++d) {
    if (!dst.out[d] || !dst.out_resid[d]) return fail(BB200_E_INVALID_ARGUMENT, "layernorm: null tensor pointer");
    if (!aligned16(dst.out[d]) || !aligned16(dst.out_resid[d])) return fail(BB200_E_MISALIGNED, "layernorm: all tensors must be 16-byte aligned");
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BB200_BF16: return dispatch<__nv_bfloat16>(x, residual, weight, bias, dst, rows, hidden, weight_is_full, bias_is_full, epsilon, s);
    case BB200_F16: return dispatch<__half>(x, residual, weight, bias, dst, rows, hidden, weight_is_full, bias_is_full, epsilon, s);
    case BB200_F32: return dispatch<float>(x, residual, weight, bias, dst, rows, hidden, weight_is_full, bias_is_full, epsilon, s);
    default: return fail(BB200_E_INVALID_ARGUMENT, "layernorm: dtype %d is not bf16/f16/f32", (int)dtype);
  }
}

extern "C" int bb200_layernorm(bb200_dtype dtype, const void* x, const void* residual, const void* weight, const void* bias,
                               void* out, void* out_resid, size_t rows, size_t hidden, int weight_is_full, int bias_is_full,
                               float epsilon, void* stream) {
  LayerNormDestinations single = {};
  single.out[0] = out;
  single.out_resid[0] = out_resid;
  single.count = 1;
  single.row_offset = 0;
  return layernorm_into(dtype, x, residual, weight, bias, single, rows, hidden, weight_is_full, bias_is_full, epsilon, stream);
}

extern "C" int bb200_layernorm_gather(bb200_dtype dtype, const void* x, const void* residual, const void* weight, const void* bias,
                                      void* const* out_destinations, void* const* out_resid_destinations, int destination_count,
                                      size_t row_offset, size_t rows, size_t hidden, int weight_is_full, int bias_is_full,
                                      float epsilon, void* stream) {
  if (!out_destinations || !out_resid_destinations || destination_count < 1 || destination_count > kMaxDestinations)
    return fail(BB200_E_INVALID_ARGUMENT, "layernorm (gather): 1..%d destination buffers are needed (got %d)", kMaxDestinations,
                destination_count);
  LayerNormDestinations all = {};
  for (int d = 0; d < destination_count; ++d) {
    all.out[d] = out_destinations[d];
    all.out_resid[d] = out_resid_destinations[d];
  }
  all.count = destination_count;
  all.row_offset = row_offset;
  return layernorm_into(dtype, x, residual, weight, bias, all, rows, hidden, weight_is_full, bias_is_full, epsilon, stream);
}

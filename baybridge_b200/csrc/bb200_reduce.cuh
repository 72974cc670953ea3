// bb200_reduce.cuh — skeletons of the reduction kernels of the b200 backend (sm_100a).
//
// A traced reduction is "map, then fold": out[kept...] = fold_op over reduced axes of f(inputs).
// The mapped value f comes from a Body (emitted from the traced dataflow graph, like the elementwise
// bodies); this header supplies the traversal, the 16-byte streaming loads, the warp/block folds
// and the three shapes a row-major tensor can be reduced in:
//   rows  [outer, inner] -> [outer]   the reduced axes are the trailing (contiguous) ones
//   cols  [outer, inner] -> [inner]   the reduced axes are the leading ones
//   all   [n] -> scalar               two launches of `rows` over a chunked view
// HBM-bound: every input element is read exactly once.
#pragma once
#include "bb200_elementwise.cuh"

namespace bb200 {

// Fold operators on the compute type; MAX/MIN keep the accumulator on ties and follow
// "lhs if lhs >= rhs else rhs" so NaN handling matches a sequential Python fold.
enum class Fold { Add, Mul, Max, Min, And, Or, Xor };

template <Fold OP, typename C> __device__ __forceinline__ C fold(C acc, C value) {
  if constexpr (OP == Fold::Add) return acc + value;
  if constexpr (OP == Fold::Mul) return acc * value;
  if constexpr (OP == Fold::Max) return acc >= value ? acc : value;
  if constexpr (OP == Fold::Min) return acc <= value ? acc : value;
  if constexpr (OP == Fold::And) return (C)((long long)acc & (long long)value);
  if constexpr (OP == Fold::Or) return (C)((long long)acc | (long long)value);
  if constexpr (OP == Fold::Xor) return (C)((long long)acc ^ (long long)value);
  return acc;
}

template <typename C> __device__ __forceinline__ C shuffle_xor(C value, int lane_mask) {
  if constexpr (sizeof(C) == 8) {
    long long bits = *reinterpret_cast<long long*>(&value);
    bits = __shfl_xor_sync(0xffffffffu, bits, lane_mask);
    return *reinterpret_cast<C*>(&bits);
  } else {
    return __shfl_xor_sync(0xffffffffu, value, lane_mask);
  }
}

// Fold across the CTA; `identity` is the value that leaves the fold unchanged for lanes without
// data (the caller passes the fold's neutral element).  Result valid in thread 0.
template <Fold OP, typename C, int THREADS> __device__ __forceinline__ C block_fold(C value, C identity, C* scratch) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value = fold<OP, C>(value, shuffle_xor(value, offset));
  if constexpr (THREADS > 32) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = value;
    __syncthreads();
    value = lane < THREADS / 32 ? scratch[lane] : identity;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value = fold<OP, C>(value, shuffle_xor(value, offset));
  }
  return value;
}

// Body interface (C = compute type):
//   static constexpr int VEC;  struct Regs;
//   void load(size_t base, Regs&) const;           issue the 16-byte loads of elements [base, base+VEC)
//   C element(const Regs&, int j) const;            mapped value of element base+j
//   C scalar(size_t i) const;                       mapped value of element i (unaligned / ragged path)

// rows: one CTA per row of `inner` elements (clipped to `total` elements overall).  Writes
// `fold(init, row values)` through Out::store(row, value).
template <Fold OP, int THREADS, typename C, typename Body, typename Out>
__device__ __forceinline__ void reduce_rows(const Body& body, const Out& out, size_t outer, size_t inner, size_t total, C init,
                                            C identity, bool vector_ok) {
  constexpr int VEC = Body::VEC;
  __shared__ C scratch[32];
  const size_t row = blockIdx.x;
  if (row >= outer) return;
  const size_t base = row * inner;
  // the last row of a chunked view of a flat tensor may be short (or empty)
  if (base + inner > total) inner = total > base ? total - base : 0;
  C acc = identity;
  if (vector_ok && (inner % VEC) == 0 && (base % VEC) == 0) {
    const size_t nvec = inner / VEC;
    size_t v = threadIdx.x;
    // two vectors in flight per thread
    for (; v + THREADS < nvec; v += 2 * THREADS) {
      typename Body::Regs r0, r1;
      body.load(base + v * VEC, r0);
      body.load(base + (v + THREADS) * VEC, r1);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc = fold<OP, C>(acc, body.element(r0, j));
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc = fold<OP, C>(acc, body.element(r1, j));
    }
    for (; v < nvec; v += THREADS) {
      typename Body::Regs r0;
      body.load(base + v * VEC, r0);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc = fold<OP, C>(acc, body.element(r0, j));
    }
  } else {
    for (size_t i = threadIdx.x; i < inner; i += THREADS) acc = fold<OP, C>(acc, body.scalar(base + i));
  }
  acc = block_fold<OP, C, THREADS>(acc, identity, scratch);
  if (threadIdx.x == 0) out.store(row, fold<OP, C>(init, acc));
}

// cols: each thread owns one column and walks rows [row_begin, row_end) of its slab; slabs
// (gridDim.y) write partial folds that a second `cols` launch over the partials combines.
template <Fold OP, typename C, typename Body, typename Out>
__device__ __forceinline__ void reduce_cols(const Body& body, const Out& out, size_t outer, size_t inner, C init, C identity) {
  const size_t col = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= inner) return;
  const size_t slabs = gridDim.y;
  const size_t rows_per_slab = (outer + slabs - 1) / slabs;
  const size_t row_begin = (size_t)blockIdx.y * rows_per_slab;
  const size_t row_end = row_begin + rows_per_slab < outer ? row_begin + rows_per_slab : outer;
  C acc0 = identity, acc1 = identity;
  size_t row = row_begin;
  for (; row + 1 < row_end; row += 2) {
    acc0 = fold<OP, C>(acc0, body.scalar(row * inner + col));
    acc1 = fold<OP, C>(acc1, body.scalar((row + 1) * inner + col));
  }
  if (row < row_end) acc0 = fold<OP, C>(acc0, body.scalar(row * inner + col));
  const C folded = fold<OP, C>(acc0, acc1);
  out.store((size_t)blockIdx.y * inner + col, slabs == 1 ? fold<OP, C>(init, folded) : folded);
}

// cols, vectorised: each thread owns VEC adjacent columns, so a row costs it one 16-byte load per
// input, and keeps eight rows in flight.  Needs inner % VEC == 0 and 16-byte aligned inputs; the scalar
// form above covers everything else.  Slabs as above.
template <Fold OP, typename C, typename Body, typename Out>
__device__ __forceinline__ void reduce_cols_vec(const Body& body, const Out& out, size_t outer, size_t inner, C init, C identity) {
  constexpr int VEC = Body::VEC;
  const size_t col = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (col >= inner) return;
  const size_t slabs = gridDim.y;
  const size_t rows_per_slab = (outer + slabs - 1) / slabs;
  const size_t row_begin = (size_t)blockIdx.y * rows_per_slab;
  const size_t row_end = row_begin + rows_per_slab < outer ? row_begin + rows_per_slab : outer;
  C acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = identity;
  size_t row = row_begin;
  constexpr int ROWS_IN_FLIGHT = 8;
  for (; row + ROWS_IN_FLIGHT - 1 < row_end; row += ROWS_IN_FLIGHT) {
    typename Body::Regs regs[ROWS_IN_FLIGHT];
#pragma unroll
    for (int k = 0; k < ROWS_IN_FLIGHT; ++k) body.load((row + k) * inner + col, regs[k]);
#pragma unroll
    for (int k = 0; k < ROWS_IN_FLIGHT; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = fold<OP, C>(acc[j], body.element(regs[k], j));
  }
  for (; row < row_end; ++row) {
    typename Body::Regs r0;
    body.load(row * inner + col, r0);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = fold<OP, C>(acc[j], body.element(r0, j));
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) out.store((size_t)blockIdx.y * inner + col + j, slabs == 1 ? fold<OP, C>(init, acc[j]) : acc[j]);
}

}  // namespace bb200

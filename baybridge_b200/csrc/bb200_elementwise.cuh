// bb200_elementwise.cuh — skeleton of every elementwise kernel of the b200 backend (sm_100a).
//
// A kernel is "N loads, a register-resident scalar expression, M stores" over a flat index
// space.  This header supplies the memory side: 128-bit coalesced streaming loads/stores, the
// grid mapping, the ragged tail and the dtype conversions.  The expression is supplied by a
// Body type: hand-written for the ahead-of-time entry points (elementwise_aot.cu) and emitted
// from a traced kernel's dataflow graph for everything else (backend/elementwise.py).
//
// HBM-bound by construction: each element is read once and written once; a thread handles
// UNROLL independent 16-byte vectors per tensor (148 SMs x 2048 threads x 16 B x tensors x UNROLL
// bytes in flight).  The callers use UNROLL = 1: full occupancy already covers HBM3e latency, and
// the smaller CTAs leave a shorter tail (measured; the figures are beside the constant in
// backend/elementwise.py).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace bb200 {

// ---- storage <-> compute conversions ------------------------------------------------------------
// 16-bit floats are widened exactly; narrowing is one round-to-nearest-even from the compute type.
template <typename C, typename S> struct Conv;
template <> struct Conv<float, float> {
  static __device__ __forceinline__ float widen(float v) { return v; }
  static __device__ __forceinline__ float narrow(float v) { return v; }
};
template <> struct Conv<double, float> {
  static __device__ __forceinline__ double widen(float v) { return (double)v; }
  static __device__ __forceinline__ float narrow(double v) { return __double2float_rn(v); }
};
template <> struct Conv<float, __nv_bfloat16> {
  static __device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 narrow(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Conv<double, __nv_bfloat16> {
  static __device__ __forceinline__ double widen(__nv_bfloat16 v) { return (double)__bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 narrow(double v) { return __double2bfloat16(v); }
};
template <> struct Conv<float, __half> {
  static __device__ __forceinline__ float widen(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half narrow(float v) { return __float2half_rn(v); }
};
template <> struct Conv<double, __half> {
  static __device__ __forceinline__ double widen(__half v) { return (double)__half2float(v); }
  static __device__ __forceinline__ __half narrow(double v) { return __double2half(v); }
};
template <typename C> struct Conv<C, int32_t> {
  static __device__ __forceinline__ C widen(int32_t v) { return (C)v; }
  static __device__ __forceinline__ int32_t narrow(C v) { return (int32_t)v; }
};
template <typename C> struct Conv<C, int64_t> {
  static __device__ __forceinline__ C widen(int64_t v) { return (C)v; }
  static __device__ __forceinline__ int64_t narrow(C v) { return (int64_t)v; }
};
template <typename C> struct Conv<C, int8_t> {
  static __device__ __forceinline__ C widen(int8_t v) { return (C)v; }
  static __device__ __forceinline__ int8_t narrow(C v) { return (int8_t)v; }
};
template <typename C> struct Conv<C, uint8_t> {  // i1: one byte per element
  static __device__ __forceinline__ C widen(uint8_t v) { return (C)(v != 0); }
  static __device__ __forceinline__ uint8_t narrow(C v) { return (uint8_t)(v != 0); }
};

// Python-style integer floor division and modulo (the CPU runtime evaluates // and % on ints).
__device__ __forceinline__ int64_t floordiv_i64(int64_t a, int64_t b) {
  int64_t q = a / b;
  return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q;
}
__device__ __forceinline__ int64_t floormod_i64(int64_t a, int64_t b) {
  int64_t r = a % b;
  return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r;
}

// ---- 16-byte vector access with streaming cache hints -------------------------------------------
// VEC elements of T form one access of VEC*sizeof(T) bytes, issued as 16-byte transactions.
template <typename T, int VEC> struct alignas(sizeof(T) * VEC >= 16 ? 16 : sizeof(T) * VEC) Pack {
  T v[VEC];
};

template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> load_stream(const T* __restrict__ p) {
  constexpr int BYTES = sizeof(T) * VEC;
  Pack<T, VEC> out;
  if constexpr (BYTES % 16 == 0) {
    const int4* src = reinterpret_cast<const int4*>(p);
    int4* dst = reinterpret_cast<int4*>(&out);
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) dst[i] = __ldcs(src + i);  // ld.global.cs: evict-first, data is used once
  } else if constexpr (BYTES == 8) {
    *reinterpret_cast<int2*>(&out) = __ldcs(reinterpret_cast<const int2*>(p));
  } else if constexpr (BYTES == 4) {
    *reinterpret_cast<int*>(&out) = __ldcs(reinterpret_cast<const int*>(p));
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out.v[i] = p[i];
  }
  return out;
}

// A vector step of an input that is only defined for elements below `bound` (a guarded load feeding zero padding):
// whole steps below the bound are ordinary vector loads, the step that straddles it reads its in-range elements one by
// one, steps past it read nothing.  Out-of-range lanes hold zero; the body substitutes the traced fallback value.
template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> load_stream_guarded(const T* __restrict__ p, size_t base, size_t bound) {
  if (base + VEC <= bound) return load_stream<T, VEC>(p + base);
  Pack<T, VEC> out;
#pragma unroll
  for (int i = 0; i < VEC; ++i) out.v[i] = base + i < bound ? p[base + i] : T();
  return out;
}

// The same access without the streaming hint, for small operands that many elements share (a row vector
// broadcast over the rows): they should stay in cache.
template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> load_shared_operand(const T* __restrict__ p) {
  Pack<T, VEC> out;
  constexpr int BYTES = sizeof(T) * VEC;
  if constexpr (BYTES % 16 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4*>(&out)[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out.v[i] = __ldg(p + i);
  }
  return out;
}

template <typename T, int VEC> __device__ __forceinline__ void store_stream(T* __restrict__ p, const Pack<T, VEC>& in) {
  constexpr int BYTES = sizeof(T) * VEC;
  if constexpr (BYTES % 16 == 0) {
    int4* dst = reinterpret_cast<int4*>(p);
    const int4* src = reinterpret_cast<const int4*>(&in);
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) __stcs(dst + i, src[i]);
  } else if constexpr (BYTES == 8) {
    __stcs(reinterpret_cast<int2*>(p), *reinterpret_cast<const int2*>(&in));
  } else if constexpr (BYTES == 4) {
    __stcs(reinterpret_cast<int*>(p), *reinterpret_cast<const int*>(&in));
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = in.v[i];
  }
}

// Destination table of the fan-out form: a rank's kernel stores its output shard into the gathered output
// buffer of every rank (its own and, through peer-mapped pointers, the others') instead of one tensor.
template <typename T> struct Destinations {
  T* p[8];
};

// ---- grid mapping ---------------------------------------------------------------------------------
// Body interface:
//   static constexpr int VEC;                                 elements per vector step (16 B of the narrowest tensor)
//   struct Regs;                                              the loaded vectors of one step
//   __device__ void load(size_t base, Regs&) const;           issue the loads of elements [base, base+VEC)
//   __device__ void compute_store(size_t base, const Regs&) const;
//   __device__ void scalar(size_t i) const;                   one element (ragged tail / unaligned pointers)
//
// Each CTA owns a contiguous tile of TILE = threads * VEC * UNROLL elements; within the tile a
// thread's UNROLL vectors are `threads * VEC` apart, so every warp-level access is a dense
// 512-byte (32 lanes x 16 B) transaction.  All UNROLL loads are issued before the first store so
// they are in flight together regardless of what the compiler can prove about aliasing.
template <int UNROLL, typename Body> __device__ __forceinline__ void flat_map(const Body& body, size_t n, bool vector_ok) {
  constexpr int VEC = Body::VEC;
  const size_t tile = (size_t)blockDim.x * VEC * UNROLL;
  const size_t tile_base = (size_t)blockIdx.x * tile;
  // Launched with programmatic stream serialisation, the next kernel of the stream may place its CTAs on SMs this
  // grid has left while this grid's last CTAs still run; such a CTA stops at `griddepcontrol.wait` until the grid before
  // it has completed and its writes are visible.  Without that launch attribute both instructions do nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tile_base >= n) return;
  if (vector_ok && tile_base + tile <= n) {
    typename Body::Regs regs[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) body.load(tile_base + ((size_t)u * blockDim.x + threadIdx.x) * VEC, regs[u]);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) body.compute_store(tile_base + ((size_t)u * blockDim.x + threadIdx.x) * VEC, regs[u]);
    return;
  }
  // last (partial) tile, or pointers that are not 16-byte aligned
  const size_t end = tile_base + tile < n ? tile_base + tile : n;
  for (size_t i = tile_base + threadIdx.x; i < end; i += blockDim.x) body.scalar(i);
}

__host__ __device__ inline unsigned flat_map_grid(size_t n, unsigned threads, int vec, int unroll) {
  const size_t tile = (size_t)threads * vec * unroll;
  return (unsigned)((n + tile - 1) / tile);
}

}  // namespace bb200

// elementwise_aot.cu — ahead-of-time instantiations of the elementwise skeleton for the C ABI:
// c = a <op> b and c = a*b + a on f32 / bf16 / f16 tensors.  Traced kernels with other bodies
// are specialised from the same skeleton at compile() time (backend/elementwise.py).
#include "bb200_elementwise.cuh"
#include "bb200_internal.h"

namespace bb200 {
namespace {

enum class Fused { Add, Sub, Mul, Div, Max, Min, MulAdd };

// Arithmetic type per storage type.  A single +,-,*,/ in f32 already equals the f64 result
// rounded once to f32, so plain f32 is exact for the binary ops; a*b+a has two roundings in
// f32, so f32 tensors evaluate it in f64 and round once (bit-equal to an f64 reference).
template <typename T, Fused OP> struct ComputeOf { using type = float; };
template <> struct ComputeOf<float, Fused::MulAdd> { using type = double; };

template <Fused OP, typename C> __device__ __forceinline__ C apply(C a, C b) {
  if constexpr (OP == Fused::Add) return a + b;
  if constexpr (OP == Fused::Sub) return a - b;
  if constexpr (OP == Fused::Mul) return a * b;
  if constexpr (OP == Fused::Div) return a / b;
  if constexpr (OP == Fused::Max) return a >= b ? a : b;  // "lhs if lhs >= rhs else rhs"
  if constexpr (OP == Fused::Min) return a <= b ? a : b;
  if constexpr (OP == Fused::MulAdd) return a * b + a;  // contraction to an FMA is exact here: one rounding either way in f64
  return a;
}

template <typename T, Fused OP> struct BinaryBody {
  using C = typename ComputeOf<T, OP>::type;
  static constexpr int VEC = 16 / sizeof(T);
  struct Regs { Pack<T, VEC> a, b; };
  const T* __restrict__ a;
  const T* __restrict__ b;
  T* __restrict__ c;
  __device__ __forceinline__ void load(size_t base, Regs& r) const {
    r.a = load_stream<T, VEC>(a + base);
    r.b = load_stream<T, VEC>(b + base);
  }
  __device__ __forceinline__ void compute_store(size_t base, const Regs& r) const {
    Pack<T, VEC> out;
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      out.v[j] = Conv<C, T>::narrow(apply<OP, C>(Conv<C, T>::widen(r.a.v[j]), Conv<C, T>::widen(r.b.v[j])));
    store_stream<T, VEC>(c + base, out);
  }
  __device__ __forceinline__ void scalar(size_t i) const {
    c[i] = Conv<C, T>::narrow(apply<OP, C>(Conv<C, T>::widen(a[i]), Conv<C, T>::widen(b[i])));
  }
};

constexpr int kThreads = 256;
constexpr int kUnroll = 1;  // as the generated kernels: one 16-byte vector per thread and stream measured fastest

template <typename T, Fused OP>
__global__ void __launch_bounds__(kThreads) binary_kernel(BinaryBody<T, OP> body, size_t n, bool vector_ok) {
  flat_map<kUnroll>(body, n, vector_ok);
}

template <typename T, Fused OP> int launch(const void* a, const void* b, void* c, size_t n, cudaStream_t stream) {
  BinaryBody<T, OP> body{static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(c)};
  const bool vector_ok = aligned16(a) && aligned16(b) && aligned16(c);
  const unsigned grid = flat_map_grid(n, kThreads, BinaryBody<T, OP>::VEC, kUnroll);
  launch_dependent(binary_kernel<T, OP>, dim3(grid), dim3(kThreads), 0, stream, body, n, vector_ok);  // flat_map waits for the kernel before
  return check_launch("elementwise kernel launch");
}

template <Fused OP> int dispatch(bb200_dtype dtype, const void* a, const void* b, void* c, size_t n, void* stream) {
  if (!a || !b || !c) return fail(BB200_E_INVALID_ARGUMENT, "elementwise: null tensor pointer");
  if (n == 0) return BB200_OK;
  if (n > ((size_t)1 << 40)) return fail(BB200_E_UNSUPPORTED_SHAPE, "elementwise: more than 2^40 elements");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BB200_F32: return launch<float, OP>(a, b, c, n, s);
    case BB200_BF16: return launch<__nv_bfloat16, OP>(a, b, c, n, s);
    case BB200_F16: return launch<__half, OP>(a, b, c, n, s);
    default: return fail(BB200_E_INVALID_ARGUMENT, "elementwise: dtype %d is not f32/bf16/f16", (int)dtype);
  }
}

}  // namespace
}  // namespace bb200

using namespace bb200;

extern "C" int bb200_elementwise_binary(bb200_binary_op op, bb200_dtype dtype, const void* a, const void* b, void* c,
                                        size_t n, void* stream) {
  switch (op) {
    case BB200_ADD: return dispatch<Fused::Add>(dtype, a, b, c, n, stream);
    case BB200_SUB: return dispatch<Fused::Sub>(dtype, a, b, c, n, stream);
    case BB200_MUL: return dispatch<Fused::Mul>(dtype, a, b, c, n, stream);
    case BB200_DIV: return dispatch<Fused::Div>(dtype, a, b, c, n, stream);
    case BB200_MAX: return dispatch<Fused::Max>(dtype, a, b, c, n, stream);
    case BB200_MIN: return dispatch<Fused::Min>(dtype, a, b, c, n, stream);
  }
  return fail(BB200_E_INVALID_ARGUMENT, "elementwise: unknown binary op %d", (int)op);
}

extern "C" int bb200_elementwise_mul_add(bb200_dtype dtype, const void* a, const void* b, void* c, size_t n, void* stream) {
  return dispatch<Fused::MulAdd>(dtype, a, b, c, n, stream);
}

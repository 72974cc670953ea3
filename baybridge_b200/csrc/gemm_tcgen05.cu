#include "bb200_internal.h"
using namespace bb200;
extern "C" int bb200_gemm_bf16(const void*, const void*, void*, int, int, int, int, int, bb200_dtype, void*) {
  return fail(BB200_E_UNSUPPORTED_SHAPE, "gemm: not built yet");
}

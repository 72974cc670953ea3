// bb200_internal.h — helpers shared by the translation units of libbb200.so (host side).
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>

#include "../../include/bb200.h"

namespace bb200 {

// Record a formatted message as this thread's last error and return `status`.
int fail(int status, const char* fmt, ...);

// Map a cudaError_t of the runtime layer to a status (0 stays 0) and record its string.
int check_runtime(cudaError_t err, const char* what);

// After a kernel launch: pick up launch-configuration errors without synchronising.
inline int check_launch(const char* what) { return check_runtime(cudaGetLastError(), what); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t dtype_bytes(bb200_dtype t) {
  switch (t) {
    case BB200_F32: case BB200_I32: return 4;
    case BB200_BF16: case BB200_F16: return 2;
    case BB200_I64: return 8;
    case BB200_I8: case BB200_I1: return 1;
  }
  return 0;
}

// Device status word for bounded waits (0 = clean).  Defined in abi_driver.cu.
int* device_status_word();

// TMA descriptor encoding through the lazily loaded driver (abi_driver.cu).
int encode_tensormap_2d(void* map_out, bb200_dtype dtype, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle);

// 3-D variant: extents (dim0 innermost), byte strides of dim1 and dim2, box extents.
int encode_tensormap_3d(void* map_out, bb200_dtype dtype, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                        int swizzle);

}  // namespace bb200

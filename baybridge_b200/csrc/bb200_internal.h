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

// Launch `kernel` with programmatic stream serialisation: its CTAs may be placed while the kernel before it on `stream`
// drains.  ONLY for kernels that run `dependent_launch_prologue()` (below) before their first global-memory access.
// A capturing stream takes the ordinary launch.
template <typename... Params, typename... Args>
inline void launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t dynamic_smem, cudaStream_t stream, Args... args) {
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  const bool capturing = cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone;
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = dynamic_smem;
  config.stream = stream;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  if (!capturing) {
    config.attrs = &attribute;
    config.numAttrs = 1;
  }
  cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);  // the caller reads the status with check_launch()
}

#ifdef __CUDACC__
// First statement of a kernel launched with launch_dependent(): lets the kernel behind this one be placed early in its
// turn, then waits until the kernel before this one has completed and its writes are visible.  Without the launch
// attribute both instructions do nothing.
__device__ __forceinline__ void dependent_launch_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

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

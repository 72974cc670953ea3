// abi_driver.cu — the thin driver shim of libbb200.so: device binding, module load, launch with
// clusters and opt-in shared memory, streams, events, staging memory, TMA descriptor encoding.
//
// libcuda.so.1 is opened lazily with dlopen (override the path with BB200_LIBCUDA, which tests
// use to inject a fake driver), so the library loads on machines without a GPU and reports
// BB200_E_NO_DRIVER only when a driver entry point is actually needed.  The CUDA runtime is
// linked statically for the ahead-of-time kernels; both layers share the device's primary
// context, which is also the one PyTorch uses.
#include <cuda.h>
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>

#include "bb200_internal.h"
#include "bb200_sm100.cuh"

namespace bb200 {

static thread_local std::string t_last_error;

int fail(int status, const char* fmt, ...) {
  char buffer[512];
  va_list args;
  va_start(args, fmt);
  vsnprintf(buffer, sizeof(buffer), fmt, args);
  va_end(args);
  t_last_error = buffer;
  return status;
}

int check_runtime(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return BB200_OK;
  return fail((int)err, "%s: %s (%s)", what, cudaGetErrorString(err), cudaGetErrorName(err));
}

// ---- lazily bound driver API ----------------------------------------------------------------------
struct DriverApi {
  void* handle = nullptr;
  CUresult (*cuInit)(unsigned) = nullptr;
  CUresult (*cuGetErrorName)(CUresult, const char**) = nullptr;
  CUresult (*cuGetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*cuDeviceGetCount)(int*) = nullptr;
  CUresult (*cuDeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*cuDeviceGetName)(char*, int, CUdevice) = nullptr;
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*cuDeviceTotalMem)(size_t*, CUdevice) = nullptr;
  CUresult (*cuDevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  CUresult (*cuCtxSetCurrent)(CUcontext) = nullptr;
  CUresult (*cuCtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*cuCtxSynchronize)() = nullptr;
  CUresult (*cuModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*cuModuleUnload)(CUmodule) = nullptr;
  CUresult (*cuModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*cuLaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
  CUresult (*cuStreamCreate)(CUstream*, unsigned) = nullptr;
  CUresult (*cuStreamDestroy)(CUstream) = nullptr;
  CUresult (*cuStreamSynchronize)(CUstream) = nullptr;
  CUresult (*cuEventCreate)(CUevent*, unsigned) = nullptr;
  CUresult (*cuEventRecord)(CUevent, CUstream) = nullptr;
  CUresult (*cuEventSynchronize)(CUevent) = nullptr;
  CUresult (*cuEventElapsedTime)(float*, CUevent, CUevent) = nullptr;
  CUresult (*cuEventDestroy)(CUevent) = nullptr;
  CUresult (*cuStreamBeginCapture)(CUstream, CUstreamCaptureMode) = nullptr;
  CUresult (*cuStreamEndCapture)(CUstream, CUgraph*) = nullptr;
  CUresult (*cuGraphInstantiateWithFlags)(CUgraphExec*, CUgraph, unsigned long long) = nullptr;
  CUresult (*cuGraphLaunch)(CUgraphExec, CUstream) = nullptr;
  CUresult (*cuGraphExecDestroy)(CUgraphExec) = nullptr;
  CUresult (*cuGraphDestroy)(CUgraph) = nullptr;
  CUresult (*cuMemAlloc)(CUdeviceptr*, size_t) = nullptr;
  CUresult (*cuMemFree)(CUdeviceptr) = nullptr;
  CUresult (*cuMemcpyHtoDAsync)(CUdeviceptr, const void*, size_t, CUstream) = nullptr;
  CUresult (*cuMemcpyDtoHAsync)(void*, CUdeviceptr, size_t, CUstream) = nullptr;
  CUresult (*cuMemsetD8Async)(CUdeviceptr, unsigned char, size_t, CUstream) = nullptr;
  CUresult (*cuMemHostAlloc)(void**, size_t, unsigned) = nullptr;
  CUresult (*cuMemFreeHost)(void*) = nullptr;
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};

static DriverApi g_api;
static std::once_flag g_api_once;
static int g_api_status = BB200_E_NO_DRIVER;
static std::string g_api_error = "driver not loaded";

template <typename Fn> static bool bind(void* handle, Fn& slot, const char* versioned, const char* plain) {
  void* symbol = versioned ? dlsym(handle, versioned) : nullptr;
  if (!symbol) symbol = dlsym(handle, plain);
  slot = reinterpret_cast<Fn>(symbol);
  return symbol != nullptr;
}

static void load_driver_once() {
  const char* override_path = getenv("BB200_LIBCUDA");
  const char* candidates[] = {override_path, "libcuda.so.1", "libcuda.so"};
  void* handle = nullptr;
  for (const char* path : candidates) {
    if (!path || !*path) continue;
    handle = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (handle) break;
    if (path == override_path) break;  // an explicit override must not fall through to the system driver
  }
  if (!handle) {
    g_api_error = "libcuda.so.1 was not found; install an NVIDIA driver or set BB200_LIBCUDA";
    return;
  }
  DriverApi& a = g_api;
  a.handle = handle;
  bool ok = true;
#define BB200_BIND(name, versioned) ok = bind(handle, a.name, versioned, #name) && ok
  BB200_BIND(cuInit, nullptr);
  BB200_BIND(cuGetErrorName, nullptr);
  BB200_BIND(cuGetErrorString, nullptr);
  BB200_BIND(cuDeviceGetCount, nullptr);
  BB200_BIND(cuDeviceGet, nullptr);
  BB200_BIND(cuDeviceGetName, nullptr);
  BB200_BIND(cuDeviceGetAttribute, nullptr);
  BB200_BIND(cuDeviceTotalMem, "cuDeviceTotalMem_v2");
  BB200_BIND(cuDevicePrimaryCtxRetain, nullptr);
  BB200_BIND(cuCtxSetCurrent, nullptr);
  BB200_BIND(cuCtxGetCurrent, nullptr);
  BB200_BIND(cuCtxSynchronize, nullptr);
  BB200_BIND(cuModuleLoadData, nullptr);
  BB200_BIND(cuModuleUnload, nullptr);
  BB200_BIND(cuModuleGetFunction, nullptr);
  BB200_BIND(cuFuncSetAttribute, nullptr);
  BB200_BIND(cuLaunchKernelEx, nullptr);
  BB200_BIND(cuStreamCreate, nullptr);
  BB200_BIND(cuStreamDestroy, "cuStreamDestroy_v2");
  BB200_BIND(cuStreamSynchronize, nullptr);
  BB200_BIND(cuEventCreate, nullptr);
  BB200_BIND(cuEventRecord, nullptr);
  BB200_BIND(cuEventSynchronize, nullptr);
  BB200_BIND(cuEventElapsedTime, nullptr);
  BB200_BIND(cuEventDestroy, "cuEventDestroy_v2");
  BB200_BIND(cuStreamBeginCapture, "cuStreamBeginCapture_v2");
  BB200_BIND(cuStreamEndCapture, nullptr);
  BB200_BIND(cuGraphInstantiateWithFlags, nullptr);
  BB200_BIND(cuGraphLaunch, nullptr);
  BB200_BIND(cuGraphExecDestroy, nullptr);
  BB200_BIND(cuGraphDestroy, nullptr);
  BB200_BIND(cuMemAlloc, "cuMemAlloc_v2");
  BB200_BIND(cuMemFree, "cuMemFree_v2");
  BB200_BIND(cuMemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2");
  BB200_BIND(cuMemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2");
  BB200_BIND(cuMemsetD8Async, nullptr);
  BB200_BIND(cuMemHostAlloc, nullptr);
  BB200_BIND(cuMemFreeHost, nullptr);
  BB200_BIND(cuTensorMapEncodeTiled, nullptr);
#undef BB200_BIND
  if (!ok) {
    g_api_error = "the CUDA driver library is missing entry points this library needs (driver older than CUDA 12?)";
    return;
  }
  CUresult init = a.cuInit(0);
  if (init != CUDA_SUCCESS) {
    const char* name = nullptr;
    a.cuGetErrorName(init, &name);
    g_api_status = (int)init;
    g_api_error = std::string("cuInit failed: ") + (name ? name : "unknown error");
    return;
  }
  g_api_status = BB200_OK;
  g_api_error.clear();
}

// Returns nullptr (and records why) when no usable driver is present.
static const DriverApi* driver() {
  std::call_once(g_api_once, load_driver_once);
  if (g_api_status != BB200_OK) {
    fail(g_api_status, "%s", g_api_error.c_str());
    return nullptr;
  }
  return &g_api;
}

static int check_driver(const DriverApi* api, CUresult result, const char* what) {
  if (result == CUDA_SUCCESS) return BB200_OK;
  const char* name = nullptr;
  const char* text = nullptr;
  api->cuGetErrorName(result, &name);
  api->cuGetErrorString(result, &text);
  return fail((int)result, "%s failed: %s (%s)", what, text ? text : "unknown", name ? name : "CUDA_ERROR_UNKNOWN");
}

#define BB200_DRIVER_OR_RETURN(api)        \
  const DriverApi* api = driver();         \
  if (!api) return g_api_status ? g_api_status : BB200_E_NO_DRIVER

// ---- device status word ---------------------------------------------------------------------------
__device__ int g_device_status = 0;

int* device_status_word() {
  int* address = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_device_status) != cudaSuccess) return nullptr;
  return address;
}

// One CTA, one mbarrier that expects an arrival nobody makes: the wait must give up after `limit_ns`, record its code
// in the status word and let the kernel return normally.
__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, int* status_word, int* returned) {
  __shared__ __align__(8) uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(sm100::smem_addr(&barrier), 1);
    sm100::fence_barrier_init();
  }
  __syncthreads();
  const bool completed = sm100::mbar_wait_limited(sm100::smem_addr(&barrier), 0, &abort_flag, status_word, BB200_WAIT_SELFTEST, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0) *returned = completed ? 2 : 1;
}

int encode_tensormap_2d(void* map_out, bb200_dtype dtype, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle) {
  BB200_DRIVER_OR_RETURN(api);
  if (!map_out || !base || !rows || !cols || !box_rows || !box_cols)
    return fail(BB200_E_INVALID_ARGUMENT, "tensormap: null pointer or zero extent");
  CUtensorMapDataType type;
  switch (dtype) {
    case BB200_BF16: type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case BB200_F16: type = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case BB200_F32: type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    case BB200_I32: type = CU_TENSOR_MAP_DATA_TYPE_INT32; break;
    case BB200_I8: case BB200_I1: type = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    default: return fail(BB200_E_INVALID_ARGUMENT, "tensormap: unsupported dtype %d", (int)dtype);
  }
  const size_t element = dtype_bytes(dtype);
  if (!aligned16(base) || (row_stride_bytes & 15u))
    return fail(BB200_E_MISALIGNED, "tensormap: base and row stride must be multiples of 16 bytes");
  if ((box_cols * element) & 15u) return fail(BB200_E_MISALIGNED, "tensormap: box row must be a multiple of 16 bytes");
  if (box_rows > 256 || box_cols > 256) return fail(BB200_E_UNSUPPORTED_SHAPE, "tensormap: box extents are limited to 256");
  static const CUtensorMapSwizzle kSwizzle[] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                                CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
  if (swizzle < 0 || swizzle > 3) return fail(BB200_E_INVALID_ARGUMENT, "tensormap: swizzle must be 0..3");
  const uint32_t swizzle_span[] = {0, 32, 64, 128};
  if (swizzle && box_cols * element > swizzle_span[swizzle])
    return fail(BB200_E_UNSUPPORTED_SHAPE, "tensormap: box row (%u B) exceeds the swizzle span (%u B)",
                (unsigned)(box_cols * element), swizzle_span[swizzle]);
  cuuint64_t dims[2] = {cols, rows};  // innermost first
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t element_strides[2] = {1, 1};
  return check_driver(api,
                      api->cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(map_out), type, 2,
                                                  const_cast<void*>(base), dims, strides, box, element_strides,
                                                  CU_TENSOR_MAP_INTERLEAVE_NONE, kSwizzle[swizzle],
                                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                      "cuTensorMapEncodeTiled");
}

int encode_tensormap_3d(void* map_out, bb200_dtype dtype, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                        int swizzle) {
  BB200_DRIVER_OR_RETURN(api);
  if (!map_out || !base || !dim0 || !dim1 || !dim2 || !box0 || !box1 || !box2)
    return fail(BB200_E_INVALID_ARGUMENT, "tensormap: null pointer or zero extent");
  if (dtype != BB200_BF16 && dtype != BB200_F16) return fail(BB200_E_INVALID_ARGUMENT, "tensormap(3d): 16-bit dtypes only");
  if (!aligned16(base) || (stride1_bytes & 15u) || (stride2_bytes & 15u))
    return fail(BB200_E_MISALIGNED, "tensormap: base and strides must be multiples of 16 bytes");
  if (swizzle != 3 || box0 * 2 != 128) return fail(BB200_E_UNSUPPORTED_SHAPE, "tensormap(3d): 128-byte rows with 128-byte swizzle only");
  if (box1 > 256 || box2 > 256) return fail(BB200_E_UNSUPPORTED_SHAPE, "tensormap: box extents are limited to 256");
  cuuint64_t dims[3] = {dim0, dim1, dim2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t element_strides[3] = {1, 1, 1};
  return check_driver(api,
                      api->cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(map_out),
                                                  dtype == BB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                                  3, const_cast<void*>(base), dims, strides, box, element_strides,
                                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                      "cuTensorMapEncodeTiled(3d)");
}

}  // namespace bb200

using namespace bb200;

extern "C" {

int bb200_abi_version(void) { return BB200_ABI_VERSION; }

const char* bb200_last_error(void) { return t_last_error.c_str(); }

int bb200_device_count(int* count) {
  if (!count) return fail(BB200_E_INVALID_ARGUMENT, "bb200_device_count: count is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuDeviceGetCount(count), "cuDeviceGetCount");
}

int bb200_init(int device) {
  BB200_DRIVER_OR_RETURN(api);
  int count = 0;
  if (int status = check_driver(api, api->cuDeviceGetCount(&count), "cuDeviceGetCount")) return status;
  if (device < 0 || device >= count)
    return fail(BB200_E_INVALID_ARGUMENT, "bb200_init: device %d is out of range (%d visible)", device, count);
  CUdevice handle;
  if (int status = check_driver(api, api->cuDeviceGet(&handle, device), "cuDeviceGet")) return status;
  CUcontext context = nullptr;
  if (int status = check_driver(api, api->cuDevicePrimaryCtxRetain(&context, handle), "cuDevicePrimaryCtxRetain"))
    return status;
  return check_driver(api, api->cuCtxSetCurrent(context), "cuCtxSetCurrent");
}

int bb200_device_info_get(int device, bb200_device_info* info) {
  if (!info) return fail(BB200_E_INVALID_ARGUMENT, "bb200_device_info_get: info is null");
  BB200_DRIVER_OR_RETURN(api);
  CUdevice handle;
  if (int status = check_driver(api, api->cuDeviceGet(&handle, device), "cuDeviceGet")) return status;
  memset(info, 0, sizeof(*info));
  info->ordinal = device;
  if (int status = check_driver(api, api->cuDeviceGetName(info->name, (int)sizeof(info->name), handle), "cuDeviceGetName"))
    return status;
  struct Query { int* slot; CUdevice_attribute attribute; } queries[] = {
      {&info->cc_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR},
      {&info->cc_minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR},
      {&info->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT},
      {&info->max_smem_per_block_optin, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN},
      {&info->l2_bytes, CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE},
      {&info->clock_khz, CU_DEVICE_ATTRIBUTE_CLOCK_RATE},
      {&info->mem_clock_khz, CU_DEVICE_ATTRIBUTE_MEMORY_CLOCK_RATE},
      {&info->mem_bus_bits, CU_DEVICE_ATTRIBUTE_GLOBAL_MEMORY_BUS_WIDTH},
  };
  for (const Query& query : queries)
    if (int status = check_driver(api, api->cuDeviceGetAttribute(query.slot, query.attribute, handle), "cuDeviceGetAttribute"))
      return status;
  size_t total = 0;
  if (int status = check_driver(api, api->cuDeviceTotalMem(&total, handle), "cuDeviceTotalMem")) return status;
  info->total_mem_bytes = total;
  return BB200_OK;
}

int bb200_module_load(const void* image, size_t image_bytes, void** module_out) {
  if (!image || !image_bytes || !module_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_module_load: null image or output");
  BB200_DRIVER_OR_RETURN(api);
  CUmodule module = nullptr;
  if (int status = check_driver(api, api->cuModuleLoadData(&module, image), "cuModuleLoadData")) return status;
  *module_out = module;
  return BB200_OK;
}

int bb200_module_unload(void* module) {
  if (!module) return fail(BB200_E_INVALID_ARGUMENT, "bb200_module_unload: module is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuModuleUnload(static_cast<CUmodule>(module)), "cuModuleUnload");
}

int bb200_get_function(void* module, const char* name, void** function_out) {
  if (!module || !name || !function_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_get_function: null argument");
  BB200_DRIVER_OR_RETURN(api);
  CUfunction function = nullptr;
  if (int status = check_driver(api, api->cuModuleGetFunction(&function, static_cast<CUmodule>(module), name),
                                "cuModuleGetFunction"))
    return status;
  *function_out = function;
  return BB200_OK;
}

int bb200_function_set_dynamic_smem(void* function, unsigned bytes) {
  if (!function) return fail(BB200_E_INVALID_ARGUMENT, "bb200_function_set_dynamic_smem: function is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api,
                      api->cuFuncSetAttribute(static_cast<CUfunction>(function),
                                              CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)bytes),
                      "cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES)");
}

static int launch_with(void* function, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3],
                       unsigned dynamic_smem_bytes, void* stream, void** params, bool dependent, const char* what) {
  if (!function || !grid || !block) return fail(BB200_E_INVALID_ARGUMENT, "%s: null function or dimensions", what);
  for (int axis = 0; axis < 3; ++axis)
    if (!grid[axis] || !block[axis]) return fail(BB200_E_INVALID_ARGUMENT, "%s: zero grid/block extent", what);
  if ((uint64_t)block[0] * block[1] * block[2] > 1024)
    return fail(BB200_E_INVALID_ARGUMENT, "%s: more than 1024 threads per block", what);
  BB200_DRIVER_OR_RETURN(api);
  CUlaunchConfig config;
  memset(&config, 0, sizeof(config));
  config.gridDimX = grid[0]; config.gridDimY = grid[1]; config.gridDimZ = grid[2];
  config.blockDimX = block[0]; config.blockDimY = block[1]; config.blockDimZ = block[2];
  config.sharedMemBytes = dynamic_smem_bytes;
  config.hStream = static_cast<CUstream>(stream);
  CUlaunchAttribute attributes[2];
  memset(attributes, 0, sizeof(attributes));
  unsigned count = 0;
  if (cluster && (cluster[0] * cluster[1] * cluster[2] > 1)) {
    for (int axis = 0; axis < 3; ++axis)
      if (!cluster[axis] || grid[axis] % cluster[axis])
        return fail(BB200_E_INVALID_ARGUMENT, "%s: grid must be a multiple of the cluster on every axis", what);
    attributes[count].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attributes[count].value.clusterDim.x = cluster[0];
    attributes[count].value.clusterDim.y = cluster[1];
    attributes[count].value.clusterDim.z = cluster[2];
    ++count;
  }
  if (dependent) {
    attributes[count].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attributes[count].value.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  if (count) {
    config.attrs = attributes;
    config.numAttrs = count;
  }
  return check_driver(api, api->cuLaunchKernelEx(&config, static_cast<CUfunction>(function), params, nullptr),
                      "cuLaunchKernelEx");
}

int bb200_launch(void* function, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3],
                 unsigned dynamic_smem_bytes, void* stream, void** params) {
  return launch_with(function, grid, block, cluster, dynamic_smem_bytes, stream, params, false, "bb200_launch");
}

int bb200_launch_dependent(void* function, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3],
                           unsigned dynamic_smem_bytes, void* stream, void** params) {
  return launch_with(function, grid, block, cluster, dynamic_smem_bytes, stream, params, true, "bb200_launch_dependent");
}

int bb200_device_synchronize(void) {
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuCtxSynchronize(), "cuCtxSynchronize");
}

int bb200_stream_synchronize(void* stream) {
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuStreamSynchronize(static_cast<CUstream>(stream)), "cuStreamSynchronize");
}

int bb200_stream_create(void** stream_out) {
  if (!stream_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_stream_create: output is null");
  BB200_DRIVER_OR_RETURN(api);
  CUstream stream = nullptr;
  if (int status = check_driver(api, api->cuStreamCreate(&stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate")) return status;
  *stream_out = stream;
  return BB200_OK;
}

int bb200_stream_destroy(void* stream) {
  if (!stream) return fail(BB200_E_INVALID_ARGUMENT, "bb200_stream_destroy: stream is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuStreamDestroy(static_cast<CUstream>(stream)), "cuStreamDestroy");
}

int bb200_event_create(void** event_out) {
  if (!event_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_event_create: output is null");
  BB200_DRIVER_OR_RETURN(api);
  CUevent event = nullptr;
  if (int status = check_driver(api, api->cuEventCreate(&event, CU_EVENT_DEFAULT), "cuEventCreate")) return status;
  *event_out = event;
  return BB200_OK;
}

int bb200_event_record(void* event, void* stream) {
  if (!event) return fail(BB200_E_INVALID_ARGUMENT, "bb200_event_record: event is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuEventRecord(static_cast<CUevent>(event), static_cast<CUstream>(stream)), "cuEventRecord");
}

int bb200_event_synchronize(void* event) {
  if (!event) return fail(BB200_E_INVALID_ARGUMENT, "bb200_event_synchronize: event is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuEventSynchronize(static_cast<CUevent>(event)), "cuEventSynchronize");
}

int bb200_event_elapsed_ms(void* start, void* stop, float* ms_out) {
  if (!start || !stop || !ms_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_event_elapsed_ms: null argument");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuEventElapsedTime(ms_out, static_cast<CUevent>(start), static_cast<CUevent>(stop)),
                      "cuEventElapsedTime");
}

int bb200_event_destroy(void* event) {
  if (!event) return fail(BB200_E_INVALID_ARGUMENT, "bb200_event_destroy: event is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuEventDestroy(static_cast<CUevent>(event)), "cuEventDestroy");
}

// ---- launch graphs: a recorded sequence of launches replayed with one driver call ------------------
int bb200_graph_capture_begin(void* stream) {
  if (!stream) return fail(BB200_E_INVALID_ARGUMENT, "bb200_graph_capture_begin: the default stream cannot record; pass a created stream");
  BB200_DRIVER_OR_RETURN(api);
  // relaxed mode: the first launch of a kernel may still load its module or size its shared memory while recording
  return check_driver(api, api->cuStreamBeginCapture(static_cast<CUstream>(stream), CU_STREAM_CAPTURE_MODE_RELAXED),
                      "cuStreamBeginCapture");
}

int bb200_graph_capture_end(void* stream, void** graph_out) {
  if (!stream || !graph_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_graph_capture_end: null stream or output");
  BB200_DRIVER_OR_RETURN(api);
  *graph_out = nullptr;
  CUgraph recorded = nullptr;
  if (int status = check_driver(api, api->cuStreamEndCapture(static_cast<CUstream>(stream), &recorded), "cuStreamEndCapture"))
    return status;
  if (!recorded) return fail(BB200_E_INVALID_ARGUMENT, "bb200_graph_capture_end: the recording was invalidated (a call that is not allowed while recording was made)");
  CUgraphExec executable = nullptr;
  const int status = check_driver(api, api->cuGraphInstantiateWithFlags(&executable, recorded, 0), "cuGraphInstantiate");
  api->cuGraphDestroy(recorded);
  if (status) return status;
  *graph_out = executable;
  return BB200_OK;
}

int bb200_graph_launch(void* graph, void* stream) {
  if (!graph) return fail(BB200_E_INVALID_ARGUMENT, "bb200_graph_launch: graph is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuGraphLaunch(static_cast<CUgraphExec>(graph), static_cast<CUstream>(stream)), "cuGraphLaunch");
}

int bb200_graph_destroy(void* graph) {
  if (!graph) return fail(BB200_E_INVALID_ARGUMENT, "bb200_graph_destroy: graph is null");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuGraphExecDestroy(static_cast<CUgraphExec>(graph)), "cuGraphExecDestroy");
}

int bb200_mem_alloc(void** device_ptr_out, size_t bytes) {
  if (!device_ptr_out || !bytes) return fail(BB200_E_INVALID_ARGUMENT, "bb200_mem_alloc: null output or zero size");
  BB200_DRIVER_OR_RETURN(api);
  CUdeviceptr pointer = 0;
  if (int status = check_driver(api, api->cuMemAlloc(&pointer, bytes), "cuMemAlloc")) return status;
  *device_ptr_out = reinterpret_cast<void*>(pointer);
  return BB200_OK;
}

int bb200_mem_free(void* device_ptr) {
  if (!device_ptr) return BB200_OK;
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuMemFree(reinterpret_cast<CUdeviceptr>(device_ptr)), "cuMemFree");
}

int bb200_memcpy_h2d(void* device_dst, const void* host_src, size_t bytes, void* stream) {
  if (!device_dst || !host_src) return fail(BB200_E_INVALID_ARGUMENT, "bb200_memcpy_h2d: null pointer");
  if (!bytes) return BB200_OK;
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api,
                      api->cuMemcpyHtoDAsync(reinterpret_cast<CUdeviceptr>(device_dst), host_src, bytes,
                                             static_cast<CUstream>(stream)),
                      "cuMemcpyHtoDAsync");
}

int bb200_memcpy_d2h(void* host_dst, const void* device_src, size_t bytes, void* stream) {
  if (!host_dst || !device_src) return fail(BB200_E_INVALID_ARGUMENT, "bb200_memcpy_d2h: null pointer");
  if (!bytes) return BB200_OK;
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api,
                      api->cuMemcpyDtoHAsync(host_dst, reinterpret_cast<CUdeviceptr>(device_src), bytes,
                                             static_cast<CUstream>(stream)),
                      "cuMemcpyDtoHAsync");
}

int bb200_memset(void* device_ptr, int byte_value, size_t bytes, void* stream) {
  if (!device_ptr) return fail(BB200_E_INVALID_ARGUMENT, "bb200_memset: null pointer");
  if (!bytes) return BB200_OK;
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api,
                      api->cuMemsetD8Async(reinterpret_cast<CUdeviceptr>(device_ptr), (unsigned char)byte_value, bytes,
                                           static_cast<CUstream>(stream)),
                      "cuMemsetD8Async");
}

int bb200_host_alloc_pinned(void** host_ptr_out, size_t bytes) {
  if (!host_ptr_out || !bytes) return fail(BB200_E_INVALID_ARGUMENT, "bb200_host_alloc_pinned: null output or zero size");
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuMemHostAlloc(host_ptr_out, bytes, 0), "cuMemHostAlloc");
}

int bb200_host_free_pinned(void* host_ptr) {
  if (!host_ptr) return BB200_OK;
  BB200_DRIVER_OR_RETURN(api);
  return check_driver(api, api->cuMemFreeHost(host_ptr), "cuMemFreeHost");
}

int bb200_tensormap_encode_2d(void* map_out, bb200_dtype dtype, const void* base, uint64_t rows, uint64_t cols,
                              uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle) {
  return encode_tensormap_2d(map_out, dtype, base, rows, cols, row_stride_bytes, box_rows, box_cols, swizzle);
}

int bb200_take_device_status(void* stream, int* status_out) {
  if (!status_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_take_device_status: output is null");
  int* word = device_status_word();
  if (!word) return fail(BB200_E_NO_DRIVER, "device status word is not addressable (no CUDA device?)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int status = check_runtime(cudaMemcpyAsync(status_out, word, sizeof(int), cudaMemcpyDeviceToHost, s), "read status"))
    return status;
  if (int status = check_runtime(cudaStreamSynchronize(s), "cudaStreamSynchronize")) return status;
  if (*status_out != 0) return check_runtime(cudaMemsetAsync(word, 0, sizeof(int), s), "clear status");
  return BB200_OK;
}

int bb200_device_status_address(void** address_out) {
  if (!address_out) return fail(BB200_E_INVALID_ARGUMENT, "bb200_device_status_address: output is null");
  int* word = device_status_word();
  if (!word) return fail(BB200_E_NO_DRIVER, "device status word is not addressable (no CUDA device?)");
  *address_out = word;
  return BB200_OK;
}

int bb200_selftest_bounded_wait(unsigned limit_us, void* stream) {
  if (limit_us == 0 || limit_us > 10000) return fail(BB200_E_INVALID_ARGUMENT, "bb200_selftest_bounded_wait: limit must be 1..10000 us");
  int* word = device_status_word();
  if (!word) return fail(BB200_E_NO_DRIVER, "device status word is not addressable (no CUDA device?)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* returned = nullptr;
  if (int status = check_runtime(cudaMallocAsync(reinterpret_cast<void**>(&returned), sizeof(int), s), "cudaMallocAsync")) return status;
  int status = check_runtime(cudaMemsetAsync(returned, 0, sizeof(int), s), "cudaMemsetAsync");
  if (!status) {
    bounded_wait_selftest_kernel<<<1, 32, 0, s>>>((unsigned long long)limit_us * 1000ull, word, returned);
    status = check_launch("bounded_wait_selftest_kernel");
  }
  int host_returned = 0;
  if (!status) status = check_runtime(cudaMemcpyAsync(&host_returned, returned, sizeof(int), cudaMemcpyDeviceToHost, s), "read back");
  if (!status) status = check_runtime(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  cudaFreeAsync(returned, s);
  if (status) return status;
  if (host_returned != 1)
    return fail(BB200_E_DEVICE_TIMEOUT, "bounded-wait self-test: the kernel %s", host_returned == 2 ? "saw a barrier phase complete that nobody arrived on"
                                                                                                : "did not reach its end");
  return BB200_OK;
}

}  // extern "C"

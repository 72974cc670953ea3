/* A stand-in for libcuda.so.1 that never touches a GPU — TEST INFRASTRUCTURE.
 *
 * libbb200.so opens the driver with dlopen and honours BB200_LIBCUDA; the tests point that variable at this
 * library to drive the driver shim on a machine without a GPU, the way upstream tests its ctypes driver wrapper
 * against a fake library (tests/test_cuda_driver_runtime.py:61, 184) and observes stream forwarding by patching
 * the driver (tests/test_backend_ptx_exec.py:3062-3145).
 *
 *   FAKE_CUDA_LOG=<path>          one line per driver call is appended there ("cuLaunchKernelEx grid=... stream=0x...")
 *   FAKE_CUDA_FAIL=name=code,...  the named entry points return that CUresult instead of succeeding
 *   FAKE_CUDA_DEVICES=<n>         what cuDeviceGetCount reports (default 1)
 *
 * "Device memory" is host memory from malloc, copies are memcpy, launches do nothing.  cuda.h maps the plain entry-point
 * names used below onto the versioned symbols (cuMemAlloc -> cuMemAlloc_v2, ...) the shim looks up first.
 */
#include <cuda.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static void record(const char* format, ...) {
  const char* path = getenv("FAKE_CUDA_LOG");
  if (!path || !*path) return;
  FILE* file = fopen(path, "a");
  if (!file) return;
  va_list args;
  va_start(args, format);
  vfprintf(file, format, args);
  va_end(args);
  fputc('\n', file);
  fclose(file);
}

/* CUresult the test asked `name` to fail with, or CUDA_SUCCESS */
static CUresult planned(const char* name) {
  const char* plan = getenv("FAKE_CUDA_FAIL");
  if (!plan) return CUDA_SUCCESS;
  size_t length = strlen(name);
  for (const char* cursor = plan; *cursor;) {
    if (!strncmp(cursor, name, length) && cursor[length] == '=') return (CUresult)atoi(cursor + length + 1);
    const char* comma = strchr(cursor, ',');
    if (!comma) break;
    cursor = comma + 1;
  }
  return CUDA_SUCCESS;
}

#define ENTER(name, ...)             \
  record(#name " " __VA_ARGS__);     \
  {                                  \
    CUresult forced = planned(#name); \
    if (forced != CUDA_SUCCESS) return forced; \
  }

static const struct { CUresult code; const char* name; const char* text; } kErrors[] = {
    {CUDA_ERROR_INVALID_VALUE, "CUDA_ERROR_INVALID_VALUE", "invalid argument"},
    {CUDA_ERROR_OUT_OF_MEMORY, "CUDA_ERROR_OUT_OF_MEMORY", "out of memory"},
    {CUDA_ERROR_NO_DEVICE, "CUDA_ERROR_NO_DEVICE", "no CUDA-capable device is detected"},
    {CUDA_ERROR_INVALID_IMAGE, "CUDA_ERROR_INVALID_IMAGE", "device kernel image is invalid"},
    {CUDA_ERROR_NOT_FOUND, "CUDA_ERROR_NOT_FOUND", "named symbol not found"},
    {CUDA_ERROR_LAUNCH_FAILED, "CUDA_ERROR_LAUNCH_FAILED", "unspecified launch failure"},
};

CUresult cuGetErrorName(CUresult error, const char** out) {
  *out = "CUDA_ERROR_UNKNOWN";
  for (size_t i = 0; i < sizeof(kErrors) / sizeof(kErrors[0]); ++i)
    if (kErrors[i].code == error) *out = kErrors[i].name;
  return CUDA_SUCCESS;
}
CUresult cuGetErrorString(CUresult error, const char** out) {
  *out = "unknown error";
  for (size_t i = 0; i < sizeof(kErrors) / sizeof(kErrors[0]); ++i)
    if (kErrors[i].code == error) *out = kErrors[i].text;
  return CUDA_SUCCESS;
}

CUresult cuInit(unsigned flags) { ENTER(cuInit, "flags=%u", flags); return CUDA_SUCCESS; }
CUresult cuDeviceGetCount(int* count) {
  ENTER(cuDeviceGetCount, "");
  const char* devices = getenv("FAKE_CUDA_DEVICES");
  *count = devices ? atoi(devices) : 1;
  return CUDA_SUCCESS;
}
CUresult cuDeviceGet(CUdevice* device, int ordinal) { ENTER(cuDeviceGet, "ordinal=%d", ordinal); *device = ordinal; return CUDA_SUCCESS; }
CUresult cuDeviceGetName(char* name, int length, CUdevice device) {
  ENTER(cuDeviceGetName, "device=%d", device);
  snprintf(name, (size_t)length, "Fake B200 #%d", device);
  return CUDA_SUCCESS;
}
CUresult cuDeviceGetAttribute(int* value, CUdevice_attribute attribute, CUdevice device) {
  (void)device;
  switch (attribute) {
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR: *value = 10; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR: *value = 0; break;
    case CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT: *value = 148; break;
    case CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN: *value = 232448; break;
    case CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE: *value = 126 << 20; break;
    default: *value = 1; break;
  }
  return CUDA_SUCCESS;
}
CUresult cuDeviceTotalMem(size_t* bytes, CUdevice device) { (void)device; *bytes = (size_t)180 << 30; return CUDA_SUCCESS; }

static CUcontext g_current;
CUresult cuDevicePrimaryCtxRetain(CUcontext* context, CUdevice device) {
  ENTER(cuDevicePrimaryCtxRetain, "device=%d", device);
  *context = (CUcontext)(size_t)(0xC0DE0000u + (unsigned)device);
  return CUDA_SUCCESS;
}
CUresult cuCtxSetCurrent(CUcontext context) { ENTER(cuCtxSetCurrent, "context=%p", (void*)context); g_current = context; return CUDA_SUCCESS; }
CUresult cuCtxGetCurrent(CUcontext* context) { *context = g_current; return CUDA_SUCCESS; }
CUresult cuCtxSynchronize(void) { ENTER(cuCtxSynchronize, ""); return CUDA_SUCCESS; }

static size_t g_modules;
CUresult cuModuleLoadData(CUmodule* module, const void* image) {
  ENTER(cuModuleLoadData, "first_bytes=%02x%02x%02x%02x context=%p", ((const unsigned char*)image)[0], ((const unsigned char*)image)[1],
        ((const unsigned char*)image)[2], ((const unsigned char*)image)[3], (void*)g_current);
  *module = (CUmodule)(0xA000 + ++g_modules);
  return CUDA_SUCCESS;
}
CUresult cuModuleUnload(CUmodule module) { ENTER(cuModuleUnload, "module=%p", (void*)module); return CUDA_SUCCESS; }
CUresult cuModuleGetFunction(CUfunction* function, CUmodule module, const char* name) {
  ENTER(cuModuleGetFunction, "module=%p name=%s", (void*)module, name);
  *function = (CUfunction)((size_t)module + 0x10000);
  return CUDA_SUCCESS;
}
CUresult cuFuncSetAttribute(CUfunction function, CUfunction_attribute attribute, int value) {
  ENTER(cuFuncSetAttribute, "function=%p attribute=%d value=%d", (void*)function, (int)attribute, value);
  return CUDA_SUCCESS;
}
CUresult cuLaunchKernelEx(const CUlaunchConfig* config, CUfunction function, void** params, void** extra) {
  (void)params, (void)extra;
  unsigned cluster[3] = {1, 1, 1};
  int dependent = 0;
  for (unsigned i = 0; i < config->numAttrs; ++i) {
    if (config->attrs[i].id == CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION) {
      cluster[0] = config->attrs[i].value.clusterDim.x;
      cluster[1] = config->attrs[i].value.clusterDim.y;
      cluster[2] = config->attrs[i].value.clusterDim.z;
    }
    if (config->attrs[i].id == CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION)
      dependent = config->attrs[i].value.programmaticStreamSerializationAllowed;
  }
  ENTER(cuLaunchKernelEx, "function=%p grid=%u,%u,%u block=%u,%u,%u cluster=%u,%u,%u smem=%u dependent=%d stream=%p",
        (void*)function, config->gridDimX, config->gridDimY, config->gridDimZ, config->blockDimX, config->blockDimY,
        config->blockDimZ, cluster[0], cluster[1], cluster[2], config->sharedMemBytes, dependent, (void*)config->hStream);
  return CUDA_SUCCESS;
}

static size_t g_streams, g_events;
CUresult cuStreamCreate(CUstream* stream, unsigned flags) { ENTER(cuStreamCreate, "flags=%u", flags); *stream = (CUstream)(0x5000 + ++g_streams); return CUDA_SUCCESS; }
CUresult cuStreamDestroy(CUstream stream) { ENTER(cuStreamDestroy, "stream=%p", (void*)stream); return CUDA_SUCCESS; }
CUresult cuStreamSynchronize(CUstream stream) { ENTER(cuStreamSynchronize, "stream=%p", (void*)stream); return CUDA_SUCCESS; }
CUresult cuEventCreate(CUevent* event, unsigned flags) { ENTER(cuEventCreate, "flags=%u", flags); *event = (CUevent)(0xE000 + ++g_events); return CUDA_SUCCESS; }
CUresult cuEventRecord(CUevent event, CUstream stream) { ENTER(cuEventRecord, "event=%p stream=%p", (void*)event, (void*)stream); return CUDA_SUCCESS; }
CUresult cuEventSynchronize(CUevent event) { ENTER(cuEventSynchronize, "event=%p", (void*)event); return CUDA_SUCCESS; }
CUresult cuEventElapsedTime(float* ms, CUevent begin, CUevent end) { (void)begin, (void)end; *ms = 0.25f; return CUDA_SUCCESS; }
CUresult cuEventDestroy(CUevent event) { ENTER(cuEventDestroy, "event=%p", (void*)event); return CUDA_SUCCESS; }

CUresult cuStreamBeginCapture(CUstream stream, CUstreamCaptureMode mode) { ENTER(cuStreamBeginCapture, "stream=%p mode=%d", (void*)stream, (int)mode); return CUDA_SUCCESS; }
CUresult cuStreamEndCapture(CUstream stream, CUgraph* graph) { ENTER(cuStreamEndCapture, "stream=%p", (void*)stream); *graph = (CUgraph)0x6001; return CUDA_SUCCESS; }
CUresult cuGraphInstantiateWithFlags(CUgraphExec* exec, CUgraph graph, unsigned long long flags) { (void)graph, (void)flags; ENTER(cuGraphInstantiateWithFlags, ""); *exec = (CUgraphExec)0x6002; return CUDA_SUCCESS; }
CUresult cuGraphLaunch(CUgraphExec exec, CUstream stream) { ENTER(cuGraphLaunch, "exec=%p stream=%p", (void*)exec, (void*)stream); return CUDA_SUCCESS; }
CUresult cuGraphExecDestroy(CUgraphExec exec) { (void)exec; ENTER(cuGraphExecDestroy, ""); return CUDA_SUCCESS; }
CUresult cuGraphDestroy(CUgraph graph) { (void)graph; ENTER(cuGraphDestroy, ""); return CUDA_SUCCESS; }

CUresult cuMemAlloc(CUdeviceptr* pointer, size_t bytes) {
  ENTER(cuMemAlloc, "bytes=%zu", bytes);
  *pointer = (CUdeviceptr)(size_t)calloc(1, bytes ? bytes : 1);
  record("cuMemAlloc.result pointer=%p", (void*)(size_t)*pointer);
  return *pointer ? CUDA_SUCCESS : CUDA_ERROR_OUT_OF_MEMORY;
}
CUresult cuMemFree(CUdeviceptr pointer) { ENTER(cuMemFree, "pointer=%p", (void*)(size_t)pointer); free((void*)(size_t)pointer); return CUDA_SUCCESS; }
CUresult cuMemcpyHtoDAsync(CUdeviceptr destination, const void* source, size_t bytes, CUstream stream) {
  ENTER(cuMemcpyHtoDAsync, "bytes=%zu stream=%p", bytes, (void*)stream);
  memcpy((void*)(size_t)destination, source, bytes);
  return CUDA_SUCCESS;
}
CUresult cuMemcpyDtoHAsync(void* destination, CUdeviceptr source, size_t bytes, CUstream stream) {
  ENTER(cuMemcpyDtoHAsync, "bytes=%zu stream=%p", bytes, (void*)stream);
  memcpy(destination, (const void*)(size_t)source, bytes);
  return CUDA_SUCCESS;
}
CUresult cuMemsetD8Async(CUdeviceptr destination, unsigned char value, size_t bytes, CUstream stream) {
  ENTER(cuMemsetD8Async, "bytes=%zu stream=%p", bytes, (void*)stream);
  memset((void*)(size_t)destination, value, bytes);
  return CUDA_SUCCESS;
}
CUresult cuMemHostAlloc(void** pointer, size_t bytes, unsigned flags) { ENTER(cuMemHostAlloc, "bytes=%zu flags=%u", bytes, flags); *pointer = calloc(1, bytes ? bytes : 1); return CUDA_SUCCESS; }
CUresult cuMemFreeHost(void* pointer) { ENTER(cuMemFreeHost, ""); free(pointer); return CUDA_SUCCESS; }

CUresult cuTensorMapEncodeTiled(CUtensorMap* map, CUtensorMapDataType type, cuuint32_t rank, void* base, const cuuint64_t* dims,
                                const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* element_strides,
                                CUtensorMapInterleave interleave, CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promotion,
                                CUtensorMapFloatOOBfill fill) {
  (void)strides, (void)element_strides, (void)interleave, (void)promotion, (void)fill;
  ENTER(cuTensorMapEncodeTiled, "type=%d rank=%u base=%p dim0=%llu box0=%u swizzle=%d", (int)type, rank, base,
        (unsigned long long)dims[0], box[0], (int)swizzle);
  memset(map, 0, sizeof(*map));
  return CUDA_SUCCESS;
}

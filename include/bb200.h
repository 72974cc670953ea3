/*
 * bb200.h — C ABI of libbb200.so, the native half of the baybridge `b200` backend.
 *
 * Plain C: pointers, sizes and ints only; no C++ or framework types cross this
 * boundary.  Every function returns an int status: 0 = success, a positive
 * value is the CUresult / cudaError_t the CUDA layer reported, a negative value
 * is one of the BB200_E_* validation codes below.  After a non-zero return,
 * bb200_last_error() gives a thread-local, human-readable description.
 * Nothing here throws, and no call falls back to host computation.
 *
 * "Replaces" lines name the interface of the upstream Python package
 * (powderluv/baybridge, paths relative to its repository root) that the entry
 * point stands in for.
 */
#ifndef BB200_H_
#define BB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BB200_ABI_VERSION 1

/* ---- status codes ---------------------------------------------------------------------- */
#define BB200_OK 0
#define BB200_E_INVALID_ARGUMENT (-1)   /* null pointer, zero/negative extent, unknown enum     */
#define BB200_E_UNSUPPORTED_SHAPE (-2)  /* shape outside what the kernel family implements      */
#define BB200_E_MISALIGNED (-3)         /* pointer or leading dimension not 16-byte aligned     */
#define BB200_E_NO_DRIVER (-4)          /* libcuda.so.1 could not be loaded / symbol missing    */
#define BB200_E_NOT_SM100 (-5)          /* the current device is not compute capability 10.x    */
#define BB200_E_DEVICE_TIMEOUT (-6)     /* a bounded in-kernel wait gave up; the context lives  */
#define BB200_E_TOO_LARGE (-7)          /* request exceeds a fixed capacity of a no-alloc entry */

/* ---- element types (names follow the IR dtype names of src/baybridge/dtypes.py:7-18) ---- */
typedef enum bb200_dtype {
  BB200_F32 = 0,
  BB200_BF16 = 1,
  BB200_F16 = 2,
  BB200_I32 = 3,
  BB200_I64 = 4,
  BB200_I8 = 5,
  BB200_I1 = 6 /* one byte per element, 0 or 1 */
} bb200_dtype;

/* ---- binary elementwise ops (scalar op names of src/baybridge/tracing.py:27-133, math.py:69-72) */
typedef enum bb200_binary_op {
  BB200_ADD = 0,
  BB200_SUB = 1,
  BB200_MUL = 2,
  BB200_DIV = 3,
  BB200_MAX = 4,
  BB200_MIN = 5
} bb200_binary_op;

/* ======================================================================================= */
/* Library / device                                                                         */
/* ======================================================================================= */

/* ABI version of the loaded library (compare with BB200_ABI_VERSION). */
int bb200_abi_version(void);

/* Thread-local description of the most recent failure on this thread ("" if none). */
const char* bb200_last_error(void);

/* Number of CUDA devices.  Replaces CudaDriver.device_count (src/baybridge/cuda_driver.py:247-250). */
int bb200_device_count(int* count);

/* Bind the calling thread to `device`: retains its primary context (shared with the CUDA
 * runtime and PyTorch) and makes it current.  Unlike upstream, any ordinal is accepted.
 * Replaces CudaDriver.ensure_primary_context (src/baybridge/cuda_driver.py:292-300). */
int bb200_init(int device);

typedef struct bb200_device_info {
  int ordinal;
  int cc_major;
  int cc_minor;
  int sm_count;
  int max_smem_per_block_optin; /* bytes */
  int l2_bytes;
  int clock_khz;
  int mem_clock_khz;
  int mem_bus_bits;
  uint64_t total_mem_bytes;
  char name[128];
} bb200_device_info;

/* Replaces CudaDriver.device_name / compute_capability (src/baybridge/cuda_driver.py:252-284). */
int bb200_device_info_get(int device, bb200_device_info* info);

/* ======================================================================================= */
/* Driver shim: module load, launch, streams, events, memory                                */
/* ======================================================================================= */

/* Load a cubin/fatbin/PTX image into the current context.
 * Replaces CudaDriver.load_module_from_ptx (src/baybridge/cuda_driver.py:327-342), which
 * accepts PTX text only. */
int bb200_module_load(const void* image, size_t image_bytes, void** module_out);

/* Replaces CudaDriver.unload_module (src/baybridge/cuda_driver.py:344-345). */
int bb200_module_unload(void* module);

/* Replaces CudaDriver.function (src/baybridge/cuda_driver.py:347-350). */
int bb200_get_function(void* module, const char* name, void** function_out);

/* Raise a function's dynamic shared-memory limit (up to 227 KB on sm_100).  No upstream
 * counterpart: its launch path is capped at the 48 KB default. */
int bb200_function_set_dynamic_smem(void* function, unsigned bytes);

/* Launch with optional thread-block-cluster dimensions (cluster = {1,1,1} or NULL for none).
 * `params` is an array of pointers to the argument values, one per kernel parameter.
 * Asynchronous on `stream` (NULL = the legacy default stream).
 * Replaces CudaDriver.launch_kernel (src/baybridge/cuda_driver.py:377-419), which has no
 * cluster support and no dynamic-smem opt-in. */
int bb200_launch(void* function, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3],
                 unsigned dynamic_smem_bytes, void* stream, void** params);

/* bb200_launch with programmatic stream serialisation (CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION): the
 * kernel's CTAs may be placed on SMs that the kernel before it on `stream` has already left, while that kernel's last
 * CTAs still run, which hides the launch latency and the ramp of a short kernel (1.6 us per launch measured).  ONLY for
 * kernels that execute `griddepcontrol.wait` before their first global-memory access — the wait returns once the kernel
 * before has completed and its writes are visible, so stream order is kept; the generated flat elementwise kernels do
 * (csrc/bb200_elementwise.cuh), and they execute `griddepcontrol.launch_dependents` first so that a dependent kernel
 * behind them may start early in turn.  After anything that is not a kernel (a copy, a memset, an event wait) the
 * launch is an ordinary one.  No upstream counterpart (upstream launches and synchronises one kernel at a time,
 * src/baybridge/cuda_driver.py:377-419). */
int bb200_launch_dependent(void* function, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3],
                           unsigned dynamic_smem_bytes, void* stream, void** params);

/* Replaces CudaDriver.synchronize / synchronize_stream (src/baybridge/cuda_driver.py:302-325). */
int bb200_device_synchronize(void);
int bb200_stream_synchronize(void* stream);

/* Create / destroy a non-blocking stream.  No upstream counterpart: upstream only forwards a stream
 * handle supplied by the caller (src/baybridge/backends/ptx_exec.py:160-171). */
int bb200_stream_create(void** stream_out);
int bb200_stream_destroy(void* stream);

/* CUDA-event timing on the launching stream (upstream times with the host clock only,
 * src/baybridge/testing.py:18-33). */
int bb200_event_create(void** event_out);
int bb200_event_record(void* event, void* stream);
int bb200_event_synchronize(void* event);
int bb200_event_elapsed_ms(void* start, void* stop, float* ms_out);
int bb200_event_destroy(void* event);

/* Launch graphs.  Between capture_begin and capture_end every launch made on `stream` (a created stream, not the
 * default one) — bb200_launch, the per-op entry points, copies and memsets — is recorded instead of executed;
 * capture_end returns an executable graph that bb200_graph_launch replays on any stream with a single driver call,
 * pointers and sizes as recorded.  Nothing may synchronise `stream` while it records.  For launch-latency-bound
 * loops of small kernels (config 1 is one).  No upstream counterpart: upstream launches and synchronises one
 * kernel at a time (src/baybridge/backends/ptx_exec.py:160-171). */
int bb200_graph_capture_begin(void* stream);
int bb200_graph_capture_end(void* stream, void** graph_out);
int bb200_graph_launch(void* graph, void* stream);
int bb200_graph_destroy(void* graph);

/* Device memory for staging host tensors.
 * Replace CudaDriver.mem_alloc / mem_free / memcpy_htod / memcpy_dtoh
 * (src/baybridge/cuda_driver.py:352-375).  Copies are asynchronous on `stream`; pass pinned
 * host memory for true overlap. */
int bb200_mem_alloc(void** device_ptr_out, size_t bytes);
int bb200_mem_free(void* device_ptr);
int bb200_memcpy_h2d(void* device_dst, const void* host_src, size_t bytes, void* stream);
int bb200_memcpy_d2h(void* host_dst, const void* device_src, size_t bytes, void* stream);
int bb200_memset(void* device_ptr, int byte_value, size_t bytes, void* stream);
int bb200_host_alloc_pinned(void** host_ptr_out, size_t bytes);
int bb200_host_free_pinned(void* host_ptr);

/* Encode a 2-D tiled TMA descriptor (CUtensorMap, 128 bytes, written to `map_out`, which must
 * be 64-byte aligned) for a row-major [rows, cols] tensor of `dtype` whose rows are
 * `row_stride_bytes` apart.  swizzle: 0 none, 1 = 32B, 2 = 64B, 3 = 128B.  No upstream
 * counterpart. */
int bb200_tensormap_encode_2d(void* map_out, bb200_dtype dtype, const void* base, uint64_t rows, uint64_t cols,
                              uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle);

/* ======================================================================================= */
/* Hot-path operators (raw device pointers; asynchronous on `stream`)                       */
/* ======================================================================================= */
/* The upstream native convention these follow is `extern "C" int launch_<kernel>(ptrs...,
 * scalars...)` returning 0 on success (src/baybridge/backends/hipcc_exec.py:31-41, 189-207;
 * src/baybridge/backends/hipkittens_exec.py:536-545, 1037-1043). */

/* c[i] = a[i] <op> b[i] for i < n; dtype f32 / bf16 / f16 (16-bit types compute in f32 with one
 * rounding at the store).  128-bit vectorised when all three pointers are 16-byte aligned.
 * Replaces the rank-1 indexed/direct binary PTX kernels (src/baybridge/backends/ptx_bridge.py:
 * 542-586, 5810-5897) — f32 only upstream. */
int bb200_elementwise_binary(bb200_binary_op op, bb200_dtype dtype, const void* a, const void* b, void* c,
                             size_t n, void* stream);

/* c[i] = a[i] * b[i] + a[i] (the fused multiply-add config), same dtype rules; the product and
 * sum are kept in f32 (f64 for f32 tensors) and rounded once.  No upstream native counterpart
 * (upstream runs it on the CPU runtime: src/baybridge/runtime.py:507-532). */
int bb200_elementwise_mul_add(bb200_dtype dtype, const void* a, const void* b, void* c, size_t n, void* stream);

/* out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * gamma, fp32 reduction, one rounding.
 * x/out: [rows, hidden] row-major; gamma: [hidden] (gamma_is_full = 0) or [rows, hidden]
 * (gamma_is_full = 1).  dtype bf16 / f16 / f32; hidden must be a multiple of 8 (16-bit) or 4
 * (f32).  Replaces launch_<kernel> of the RMSNorm template
 * (src/baybridge/backends/hipkittens_exec.py:1105-1176; semantics src/baybridge/frontend.py:3828-3852). */
int bb200_rmsnorm(bb200_dtype dtype, const void* x, const void* gamma, void* out, size_t rows, size_t hidden,
                  int gamma_is_full, float epsilon, void* stream);

/* bb200_rmsnorm fused with the all-gather of its output across the GPUs of one box: this GPU's [rows, hidden]
 * result is the row block starting at `row_offset` of a taller tensor of which every GPU holds a copy, and each
 * normalised vector is stored into all `destination_count` (1..8) copies — out_destinations[d] is the base of
 * copy d (the GPU's own buffer or a peer-mapped pointer; ordinary 16-byte stores over NVLink).  The caller
 * still needs a barrier across the GPUs before the gathered tensor is read.  Other arguments as bb200_rmsnorm.
 * No upstream counterpart (upstream is single-device: src/baybridge/backends/cuda_driver.py:292-300). */
int bb200_rmsnorm_gather(bb200_dtype dtype, const void* x, const void* gamma, void* const* out_destinations,
                         int destination_count, size_t row_offset, size_t rows, size_t hidden, int gamma_is_full,
                         float epsilon, void* stream);

/* mixed = x + residual; out_resid = mixed; out = (mixed - mean) / sqrt(var + eps) * weight + bias, with mean and
 * (biased) variance over the last axis in fp32 and one rounding per output.  x/residual/out/out_resid: [rows, hidden]
 * row-major; weight and bias: [hidden] (…_is_full = 0) or [rows, hidden] (…_is_full = 1).  dtype bf16 / f16 / f32;
 * hidden a multiple of 8 (16-bit) or 4 (f32) and at most 32768 (16-bit) / 16384 (f32).  Replaces launch_<kernel> of
 * the LayerNorm template (src/baybridge/backends/hipkittens_exec.py:1046-1103; semantics
 * src/baybridge/frontend.py:3754-3793). */
int bb200_layernorm(bb200_dtype dtype, const void* x, const void* residual, const void* weight, const void* bias, void* out,
                    void* out_resid, size_t rows, size_t hidden, int weight_is_full, int bias_is_full, float epsilon,
                    void* stream);

/* bb200_layernorm fused with the all-gather of both outputs across the GPUs of one box: this GPU's rows are the block
 * starting at `row_offset` of taller out / out_resid tensors of which every GPU holds a copy, and every output vector
 * is stored into all `destination_count` (1..8) copies (own buffers or peer-mapped pointers; ordinary 16-byte stores
 * over NVLink).  The caller still needs a barrier across the GPUs before the gathered tensors are read.  Other
 * arguments as bb200_layernorm.  No upstream counterpart (upstream is single-device:
 * src/baybridge/backends/cuda_driver.py:292-300). */
int bb200_layernorm_gather(bb200_dtype dtype, const void* x, const void* residual, const void* weight, const void* bias,
                           void* const* out_destinations, void* const* out_resid_destinations, int destination_count,
                           size_t row_offset, size_t rows, size_t hidden, int weight_is_full, int bias_is_full,
                           float epsilon, void* stream);

/* C[m, n] = sum_k A'[m, k] * B'[k, n]; A' = A or A^T, B' = B or B^T per the transpose flags;
 * A, B bf16 row-major as stored ([m,k] or [k,m]; [k,n] or [n,k]); C row-major [m, n] of
 * c_dtype bf16 or f32; fp32 accumulation on tcgen05 tensor cores; C is overwritten.  Every layout is
 * read in place except A stored [k, m] with m not a multiple of 8, which is first transposed into a
 * stream-ordered workspace taken from the driver.  Problems with few output tiles and a deep k are split along k
 * into fp32 partial products (a second stream-ordered workspace of at most 16 * m * n floats) that a second kernel folds.
 * Replaces launch_<kernel> of the GEMM template (src/baybridge/backends/hipkittens_exec.py:
 * 994-1044; semantics src/baybridge/frontend.py:3684-3716). */
int bb200_gemm_bf16(const void* a, const void* b, void* c, int m, int n, int k, int transpose_a, int transpose_b,
                    bb200_dtype c_dtype, void* stream);

/* Same contract and same kernels as bb200_gemm_bf16, for callers that must not allocate device memory
 * while they run — a server whose own pools already fill the GPU, a framework whose allocator has to
 * stay the sole owner of device memory, a latency-critical loop that cannot afford a driver
 * allocation stalling or failing late.  bb200_gemm_bf16 takes a stream-ordered workspace from the
 * driver when A is stored [k, m] with m not a multiple of 8; this entry point puts that transposed
 * copy of A into a 32 MiB buffer built into the library instead, and performs no cudaMalloc /
 * cudaFree / pool operation of any kind; it also never splits a problem along k (that needs a workspace), so small
 * outputs with a deep k run as one work item per tile.  Limits and rules:
 *   - with transpose_a != 0 and m % 8 != 0, m*k must not exceed 16,777,216 elements (32 MiB of bf16);
 *     larger requests return BB200_E_TOO_LARGE.  In every other case the buffer is not used and any
 *     size is accepted.
 *   - the buffer exists once per GPU and every call uses it, so two calls whose GPU work may overlap
 *     (different streams or threads) must be serialised by the caller; it keeps the previous call's
 *     contents between calls, which is harmless because each call overwrites what it reads.
 *   - the first call on each device looks up the buffer's device address (that device must be
 *     current); make that first call before starting any stream capture.
 * This entry point has no counterpart in the upstream package. */
int bb200_gemm_bf16_noalloc(const void* a, const void* b, void* c, int m, int n, int k, int transpose_a,
                            int transpose_b, bb200_dtype c_dtype, void* stream);

/* bb200_gemm_bf16 fused with the all-gather of its output across the GPUs of one box.  Each GPU multiplies its
 * own row block A_r [m, k] (B is the same everywhere) and the full result is the row-wise concatenation
 * C = [C_0; C_1; ...] that every GPU wants a copy of.  Instead of writing C_r locally and all-gathering
 * afterwards, the epilogue stores every tile of C_r into all `destination_count` copies of C — the GPU's own
 * buffer and, through peer-mapped pointers (CUDA IPC / symmetric memory; ordinary stores over NVLink), the
 * others' — at row `row_offset` (= r * m).  c_destinations[d] is the base of copy d, a row-major
 * [rows >= row_offset + m, n] matrix of c_dtype; 1 <= destination_count <= 8.  The caller still needs a
 * barrier across the GPUs before anyone reads C.  Other arguments as bb200_gemm_bf16.
 * No upstream counterpart (upstream is single-device: src/baybridge/backends/cuda_driver.py:292-300). */
int bb200_gemm_bf16_gather(const void* a, const void* b, void* const* c_destinations, int destination_count, int row_offset,
                           int m, int n, int k, int transpose_a, int transpose_b, bb200_dtype c_dtype, void* stream);

/* Softmax attention forward.  q/out: [batch, seq, heads, head_dim]; k/v: [batch, seq, kv_heads,
 * head_dim] (heads % kv_heads == 0), all bf16 row-major; lse: fp32 [batch, heads, seq]
 * (identical memory layout to [batch, heads, 1, seq]), natural log.  Scale is fixed at
 * 1/sqrt(head_dim).  causal != 0 masks key > query.  For head_dim 64 and 128 the kernel is persistent and draws its
 * work from a 4-byte counter inside the library that the call zeroes on `stream` first (one of 256, taken in turn, so
 * calls whose GPU work overlaps do not share one unless more than 256 are in flight); no device memory is allocated.
 * Limits that follow from the counter pool: (1) more than 256 attention launches in flight at once on one GPU (for
 * example on many streams) may share a counter, and two launches sharing one skip or repeat work items — keep at
 * most 256 unfinished calls per GPU; (2) a call recorded into a launch graph keeps the counter it drew when it was
 * recorded, so do not replay one recorded graph concurrently with itself, and do not let a replay overlap with more
 * than 255 newer live calls.
 * Replaces launch_<kernel> of the attention templates (src/baybridge/backends/hipkittens_exec.py:
 * 1178-1335; semantics src/baybridge/frontend.py:3877-3937). */
int bb200_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int seq,
                        int heads, int kv_heads, int head_dim, int causal, void* stream);

/* bb200_attention_fwd fused with the all-gather of its outputs across the GPUs of one box: this GPU's `batch`
 * sequences are the block starting at `batch_offset` of a larger batch of which every GPU holds a copy of out
 * ([total_batch, seq, heads, head_dim] bf16) and lse ([total_batch, heads, seq] fp32).  Each finished output
 * row and lse value is stored into all `destination_count` (1..8) copies — out_destinations[d] /
 * lse_destinations[d] are the bases of copy d (the GPU's own buffers or peer-mapped pointers; whole rows leave
 * as contiguous 16-byte stores over NVLink).  head_dim 64 or 128 only.  The caller still needs a barrier across
 * the GPUs before the gathered tensors are read.  Other arguments as bb200_attention_fwd.
 * No upstream counterpart (upstream is single-device: src/baybridge/backends/cuda_driver.py:292-300). */
int bb200_attention_fwd_gather(const void* q, const void* k, const void* v, void* const* out_destinations,
                               float* const* lse_destinations, int destination_count, int batch_offset, int batch,
                               int seq, int heads, int kv_heads, int head_dim, int causal, void* stream);

/* Kernels with bounded device-side waits record a give-up in a per-device status word.  This
 * reads and clears it: *status_out = 0 if no wait timed out since the last call.  Synchronises
 * `stream` first.  No upstream counterpart (its generated kernels never wait on one another). */
int bb200_take_device_status(void* stream, int* status_out);

/* Device address of the current device's status word, for kernels that are loaded through bb200_module_load and want
 * to record a code there themselves (the bounds-checking debug build of generated elementwise kernels does: codes 301 /
 * 302 = a load / a store whose traced index fell outside its tensor).  No upstream counterpart: upstream's generated
 * kernels skip out-of-range accesses silently (src/baybridge/backends/ptx_bridge.py:5846-5847) and its CPU runtime
 * raises IndexError. */
int bb200_device_status_address(void** address_out);

/* Status-word code written by the self-test below (kernels use codes 100 and up). */
#define BB200_WAIT_SELFTEST 99

/* Diagnostic: launches one CTA that waits, through the same bounded wait every kernel of this library uses, on a
 * barrier nobody arrives on, with a limit of `limit_us` microseconds (1..10000) instead of the kernels' 1 s.  The
 * wait gives up, the kernel returns normally and the device status word holds BB200_WAIT_SELFTEST until
 * bb200_take_device_status reads it; the context stays usable.  Returns BB200_OK when exactly that happened.
 * Synchronises `stream`.  It exercises the path by which a launcher learns of an abandoned wait — the analogue of a
 * native launch returning non-zero upstream (src/baybridge/backends/hipcc_exec.py:181-182) — without faulting. */
int bb200_selftest_bounded_wait(unsigned limit_us, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BB200_H_ */

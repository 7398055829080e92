/* ullm_cuda.h — versioned C ABI of the CUDA (sm_100a) quantised-linear backend.
 *
 * This is the CUDA sibling of the reference's HIP boundary and keeps its
 * conventions (reference file:line given beside each group):
 *   - every function returns ullm_status_t and never throws across the boundary;
 *   - the caller owns an optional error sink; message_length is always the
 *     untruncated length and a truncated message turns the return value into
 *     ULLM_STATUS_BUFFER_TOO_SMALL (include/ullm/hip.h:48-63);
 *   - validation order is: sink, then the versioned struct, then arguments
 *     (native/hip/src/hip_stub.cpp:43-118);
 *   - extensible structs start with struct_size + abi_version and end with
 *     reserved words that must be zero;
 *   - handles are opaque and never dereferenced by callers (hip.h:40-46);
 *   - host data is copied during the call; the library keeps no pointer into
 *     caller memory after return (native/hip/src/hip_evidence_runtime.hip.cpp:618-620);
 *   - completion = submit -> wait(timeout_ms) -> destroy; wait polls, it never
 *     blocks without a deadline; a completion is consumed by wait, whatever the outcome
 *     (native/hip/src/evidence_abi.h:48-59, hip_evidence_runtime.hip.cpp:508-535, :691-716);
 *   - no destructor blocks on the device: what may still be in use is retired in the
 *     background once its completion is proven, and never freed before that
 *     (hip_evidence_runtime.hip.cpp:77-103, :151-257);
 *   - there is no CPU fallback: without a usable sm_100 device every compute
 *     entry returns ULLM_STATUS_CUDA_UNAVAILABLE
 *     (native/hip/src/hip_evidence_stub.cpp:103-127).
 * The header is self-contained C99 / C++11.
 */
#ifndef ULLM_CUDA_H
#define ULLM_CUDA_H

#include <stdint.h>

/* export marker, the counterpart of ULLM_HIP_API (include/ullm/hip.h:6-14) */
#if defined(__GNUC__)
#define ULLM_CUDA_API __attribute__((visibility("default")))
#else
#define ULLM_CUDA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define ULLM_CUDA_ABI_VERSION UINT32_C(1)
#define ULLM_CUDA_LIBRARY_VERSION_MAJOR UINT32_C(0)
#define ULLM_CUDA_LIBRARY_VERSION_MINOR UINT32_C(1)
#define ULLM_CUDA_LIBRARY_VERSION_PATCH UINT32_C(0)

/* ---- status codes: 0-7 are the reference's public codes (hip.h:21-30), 8-12 its
 * private evidence codes (evidence_abi.h:13-17); 13+ are new. ------------------- */
#ifndef ULLM_STATUS_OK
typedef uint32_t ullm_status_t;
#define ULLM_STATUS_OK UINT32_C(0)
#define ULLM_STATUS_INVALID_ARGUMENT UINT32_C(1)
#define ULLM_STATUS_BUFFER_TOO_SMALL UINT32_C(2)
#define ULLM_STATUS_UNSUPPORTED UINT32_C(3)
#define ULLM_STATUS_INVALID_ABI_VERSION UINT32_C(5)
#define ULLM_STATUS_RESERVED_NONZERO UINT32_C(6)
#define ULLM_STATUS_INTERNAL_ERROR UINT32_C(7)
#endif
#define ULLM_STATUS_CUDA_UNAVAILABLE UINT32_C(4) /* same slot as ULLM_STATUS_HIP_UNAVAILABLE */
#define ULLM_STATUS_CUDA_TIMEOUT UINT32_C(8)
#define ULLM_STATUS_CUDA_INVALID_HANDLE UINT32_C(9)
#define ULLM_STATUS_CUDA_ZERO_DISPATCH UINT32_C(10)
#define ULLM_STATUS_CUDA_RUNTIME_ERROR UINT32_C(11)
#define ULLM_STATUS_CUDA_DISPATCH_CONTRACT UINT32_C(12)
#define ULLM_STATUS_CUDA_OUT_OF_MEMORY UINT32_C(13)
#define ULLM_STATUS_CUDA_OUT_OF_RANGE UINT32_C(14)   /* a tensor span leaves its buffer */
#define ULLM_STATUS_CUDA_COMM_ERROR UINT32_C(15)     /* NCCL missing or failed */
#define ULLM_STATUS_CUDA_DEVICE_FLAGGED UINT32_C(16) /* a kernel gave up a bounded wait */

#define ULLM_BACKEND_CUDA UINT32_C(2) /* next id after ULLM_BACKEND_HIP = 1 (hip.h:32) */

/* physical scalar types, numbered like ullm-core's DType (crates/ullm-core/src/dtype.rs:6-16) */
#define ULLM_CUDA_DTYPE_BF16 UINT32_C(0)
#define ULLM_CUDA_DTYPE_F16 UINT32_C(1)
#define ULLM_CUDA_DTYPE_F32 UINT32_C(2)
#define ULLM_CUDA_DTYPE_F8E4M3FN UINT32_C(3)
#define ULLM_CUDA_DTYPE_I8 UINT32_C(7)
#define ULLM_CUDA_DTYPE_U8 UINT32_C(8)

/* storage encodings, the additive siblings of Encoding::Nvfp4 (dtype.rs:56-66) */
#define ULLM_CUDA_ENCODING_UNQUANTIZED UINT32_C(0)
#define ULLM_CUDA_ENCODING_NVFP4 UINT32_C(1) /* u8 [N,K/2] e2m1 pairs + f16 [N,K/16] block scales + one f32 tensor scale;
                                                quantise / dequantise and the decode linear (M <= 8); no tensor-core path */
#define ULLM_CUDA_ENCODING_AQ4 UINT32_C(2)   /* u8 [N,K/2] nibbles + f16 [N,K/group] scales */
#define ULLM_CUDA_ENCODING_FP8_CHANNEL UINT32_C(3) /* e4m3fn [N,K] + f32 [N] scales */

#define ULLM_CUDA_AQ4_GROUP UINT32_C(128)
#define ULLM_CUDA_NVFP4_BLOCK UINT32_C(16)

/* opaque handles (hip.h:40-46) */
typedef struct ullm_cuda_context_t ullm_cuda_context_t;
typedef struct ullm_cuda_queue_t ullm_cuda_queue_t;
typedef struct ullm_cuda_buffer_t ullm_cuda_buffer_t;
typedef struct ullm_cuda_completion_t ullm_cuda_completion_t;
typedef struct ullm_cuda_graph_t ullm_cuda_graph_t;
typedef struct ullm_cuda_comm_t ullm_cuda_comm_t;
typedef struct ullm_cuda_stack_t ullm_cuda_stack_t;
typedef struct ullm_cuda_prepared_t ullm_cuda_prepared_t;
typedef struct ullm_cuda_event_t ullm_cuda_event_t;

/* identical layout to ullm_error_sink_t (hip.h:48-55): 48 bytes, align 8 */
typedef struct ullm_cuda_error_sink_t {
  uint32_t struct_size;
  uint32_t abi_version;
  char *message;
  uint64_t message_capacity; /* includes the NUL */
  uint64_t message_length;   /* required length without the NUL, even when truncated */
  uint64_t reserved[2];
} ullm_cuda_error_sink_t;

typedef struct ullm_cuda_version_info_t { /* hip.h:76-83 */
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t major;
  uint32_t minor;
  uint32_t patch;
  uint32_t reserved[3];
} ullm_cuda_version_info_t;

typedef struct ullm_cuda_backend_probe_result_t { /* hip.h:85-92, extended */
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t backend;
  uint32_t available;            /* 1 when at least one sm_100 device is usable */
  uint32_t cuda_runtime_present; /* 1 when the CUDA runtime answered at all */
  uint32_t device_count;
  uint32_t sm_major; /* of device 0 */
  uint32_t sm_minor;
  uint32_t sm_count;
  uint32_t l2_bytes_mib;
  uint64_t global_memory_bytes;
  uint32_t reserved[4];
} ullm_cuda_backend_probe_result_t;

typedef struct ullm_cuda_context_probe_result_t { /* hip.h:94-100 */
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t context_present;
  uint32_t cuda_available;
  uint32_t device_ordinal;
  uint32_t reserved[3];
} ullm_cuda_context_probe_result_t;

/* A span inside a device buffer.  Every op checks offset + bytes against the
 * buffer size on the host before launching anything. */
typedef struct ullm_cuda_tensor_t {
  ullm_cuda_buffer_t *buffer;
  uint64_t offset_bytes;
} ullm_cuda_tensor_t;

/* A quantised weight W[N,K] (row n = output channel, K contiguous). */
typedef struct ullm_cuda_weight_t {
  uint32_t encoding;   /* ULLM_CUDA_ENCODING_AQ4 | ULLM_CUDA_ENCODING_FP8_CHANNEL | ULLM_CUDA_ENCODING_NVFP4 */
  uint32_t group_size; /* 128 for AQ4; 0 for FP8_CHANNEL; 16 for NVFP4 */
  uint64_t n;
  uint64_t k;
  ullm_cuda_tensor_t values; /* AQ4 / NVFP4: u8 [N,K/2]; FP8: e4m3fn [N,K] */
  ullm_cuda_tensor_t scales; /* AQ4: f16 [N,K/128]; FP8: f32 [N]; NVFP4: f16 [N,K/16], then at the next 16-byte
                                boundary one f32 tensor scale (16-byte aligned span of that size + 4 bytes) */
} ullm_cuda_weight_t;

/* ---- version / probe: the CUDA counterparts of hip.h:106-121 ---------------- */
ULLM_CUDA_API ullm_status_t ullm_cuda_get_abi_version(uint32_t *abi_version, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_query_version(ullm_cuda_version_info_t *version, ullm_cuda_error_sink_t *error_sink);
/* ULLM_STATUS_OK with available=1 on a usable sm_100 device; ULLM_STATUS_CUDA_UNAVAILABLE
 * (result still filled) otherwise; ULLM_STATUS_UNSUPPORTED for any other backend id. */
ULLM_CUDA_API ullm_status_t ullm_cuda_backend_probe(uint32_t backend, ullm_cuda_backend_probe_result_t *result,
                                      ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_context_probe(const ullm_cuda_context_t *context,
                                      ullm_cuda_context_probe_result_t *result,
                                      ullm_cuda_error_sink_t *error_sink);

/* ---- context / queue / buffer / completion.  Replaces the per-request stream,
 * event and buffer lifecycle of native/hip/src/hip_evidence_runtime.hip.cpp:53-71,
 * :585-659 with objects that are created once and reused. ---------------------- */
ULLM_CUDA_API ullm_status_t ullm_cuda_context_create(uint32_t device_ordinal, ullm_cuda_context_t **context,
                                       ullm_cuda_error_sink_t *error_sink);
/* Fails with ULLM_STATUS_INVALID_ARGUMENT while the context still owns queues, buffers, graphs, comms or
 * stacks; an object destroyed while its queue was busy counts as owned until its background retirement ends. */
ULLM_CUDA_API ullm_status_t ullm_cuda_context_destroy(ullm_cuda_context_t **context, ullm_cuda_error_sink_t *error_sink);
/* Limit of every device-side wait of kernels launched for this context afterwards (the fused all-reduce's
 * wait for a peer's partial sums, the GEMM's pipeline barriers): 1 .. 600000 ms, default 20000.  A wait that
 * runs out makes its kernel return; everything queued behind it on the context returns without waiting, and
 * the next ullm_cuda_completion_wait reports ULLM_STATUS_CUDA_DEVICE_FLAGGED (results are not valid). */
ULLM_CUDA_API ullm_status_t ullm_cuda_context_set_wait_limit(ullm_cuda_context_t *context, uint32_t limit_ms,
                                               ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_queue_create(ullm_cuda_context_t *context, ullm_cuda_queue_t **queue,
                                     ullm_cuda_error_sink_t *error_sink);
/* Returns at once.  The stream and the queue's staging memory are released when the queue's last work is
 * observed complete (immediately if it already is); the handle is dead either way. */
ULLM_CUDA_API ullm_status_t ullm_cuda_queue_destroy(ullm_cuda_queue_t **queue, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_buffer_alloc(ullm_cuda_context_t *context, uint64_t size_bytes,
                                     ullm_cuda_buffer_t **buffer, ullm_cuda_error_sink_t *error_sink);
/* Returns at once.  The memory is freed when every queue of the context that was busy at the time of the
 * call has finished the work it had then (immediately if all were idle). */
ULLM_CUDA_API ullm_status_t ullm_cuda_buffer_free(ullm_cuda_buffer_t **buffer, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_buffer_size(const ullm_cuda_buffer_t *buffer, uint64_t *size_bytes,
                                    ullm_cuda_error_sink_t *error_sink);
/* Synchronous with respect to the caller: the bytes have left / reached host
 * memory when the call returns; ordered after earlier work on the queue. */
ULLM_CUDA_API ullm_status_t ullm_cuda_buffer_upload(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t dst, const void *host_src,
                                      uint64_t size_bytes, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_buffer_download(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t src, void *host_dst,
                                        uint64_t size_bytes, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_buffer_fill(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t dst, uint8_t value,
                                    uint64_t size_bytes, ullm_cuda_error_sink_t *error_sink);
/* Records a completion point on the queue (an event with timing).  The handle is consumed by
 * ullm_cuda_completion_wait.  Refused with ULLM_STATUS_CUDA_RUNTIME_ERROR while too many destroyed objects
 * still wait for proof that the device has finished with them (at most 8), or after one such proof failed. */
ULLM_CUDA_API ullm_status_t ullm_cuda_queue_signal(ullm_cuda_queue_t *queue, ullm_cuda_completion_t **completion,
                                     ullm_cuda_error_sink_t *error_sink);

typedef struct ullm_cuda_completion_result_t { /* evidence_abi.h:27-40 */
  uint32_t struct_size;
  uint32_t abi_version;
  uint64_t dispatch_count; /* kernels launched on the queue since the previous signal */
  uint64_t copy_count;     /* cudaMemcpyAsync transfers since the previous signal */
  uint32_t selected_backend; /* always ULLM_BACKEND_CUDA */
  uint32_t fallback_used;    /* always 0 */
  uint32_t terminal;
  uint32_t device_flags; /* non-zero when a kernel recorded a bounded-wait expiry */
  uint32_t reserved[4];
} ullm_cuda_completion_result_t;

/* timeout_ms == 0 is a single poll (hip_evidence_runtime.hip.cpp:508-535).
 * The handle is consumed by EVERY outcome, ULLM_STATUS_CUDA_TIMEOUT included (hip_evidence_runtime.hip.cpp:691-716:
 * "a caller cannot retry"); a later use returns ULLM_STATUS_CUDA_INVALID_HANDLE.  To poll without consuming,
 * use ullm_cuda_completion_query.  result may be NULL. */
ULLM_CUDA_API ullm_status_t ullm_cuda_completion_wait(ullm_cuda_completion_t *completion, uint32_t timeout_ms,
                                        ullm_cuda_completion_result_t *result,
                                        ullm_cuda_error_sink_t *error_sink);
/* Milliseconds of device time between two completions that have both been
 * reached (the handles stay valid: use this BEFORE a wait consumes them; ullm_cuda_completion_query tells
 * when they have been reached). */
ULLM_CUDA_API ullm_status_t ullm_cuda_completion_elapsed_ms(ullm_cuda_completion_t *start, ullm_cuda_completion_t *end,
                                              float *milliseconds, ullm_cuda_error_sink_t *error_sink);
/* Poll without consuming: OK when reached, ULLM_STATUS_CUDA_TIMEOUT when not. */
ULLM_CUDA_API ullm_status_t ullm_cuda_completion_query(ullm_cuda_completion_t *completion, uint32_t timeout_ms,
                                         ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_completion_destroy(ullm_cuda_completion_t **completion,
                                           ullm_cuda_error_sink_t *error_sink);

/* Stream capture into a replayable graph: everything enqueued on the queue
 * between begin and end is recorded instead of run. */
ULLM_CUDA_API ullm_status_t ullm_cuda_queue_capture_begin(ullm_cuda_queue_t *queue, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_queue_capture_end(ullm_cuda_queue_t *queue, ullm_cuda_graph_t **graph,
                                          ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_graph_launch(ullm_cuda_graph_t *graph, ullm_cuda_queue_t *queue,
                                     ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_graph_destroy(ullm_cuda_graph_t **graph, ullm_cuda_error_sink_t *error_sink);

/* ---- synthetic data (counter-based, bit-identical to the CPU oracle) ---------- */
/* fp32 out[i] = std * z(seed, tensor_id, first_element + i) */
ULLM_CUDA_API ullm_status_t ullm_cuda_synth_weights(ullm_cuda_queue_t *queue, uint64_t seed, uint64_t tensor_id,
                                      uint64_t first_element, uint64_t count, float std,
                                      ullm_cuda_tensor_t out_f32, ullm_cuda_error_sink_t *error_sink);
/* bf16 out[i] = bf16_rne(z(...)) */
ULLM_CUDA_API ullm_status_t ullm_cuda_synth_activations(ullm_cuda_queue_t *queue, uint64_t seed, uint64_t tensor_id,
                                          uint64_t first_element, uint64_t count, ullm_cuda_tensor_t out_bf16,
                                          ullm_cuda_error_sink_t *error_sink);

/* ---- quantisation, packing, unpacking (bit-exact against the oracle).  The
 * reference has no counterpart: these fill the encodings that
 * crates/ullm-core/src/dtype.rs:56-122 only describes. -------------------------- */
/* fp32 W[N,K] -> weight.values / weight.scales.  K % group == 0, else UNSUPPORTED. */
ULLM_CUDA_API ullm_status_t ullm_cuda_quantize(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t src_f32,
                                 const ullm_cuda_weight_t *weight, ullm_cuda_error_sink_t *error_sink);
/* AQ4 only: nibbles -> int8 q[N,K] in [-8,7]. */
ULLM_CUDA_API ullm_status_t ullm_cuda_aq4_unpack(ullm_cuda_queue_t *queue, const ullm_cuda_weight_t *weight,
                                   ullm_cuda_tensor_t out_i8, ullm_cuda_error_sink_t *error_sink);
/* AQ4 only: int8 q[N,K] -> nibbles (scales untouched). */
ULLM_CUDA_API ullm_status_t ullm_cuda_aq4_pack(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t src_i8,
                                 const ullm_cuda_weight_t *weight, ullm_cuda_error_sink_t *error_sink);
/* W'[N,K] as out_dtype (F32 exact; BF16 rounds to nearest even). */
ULLM_CUDA_API ullm_status_t ullm_cuda_dequantize(ullm_cuda_queue_t *queue, const ullm_cuda_weight_t *weight,
                                   ullm_cuda_tensor_t out, uint32_t out_dtype,
                                   ullm_cuda_error_sink_t *error_sink);

/* ---- weights from a safetensors file, quantised on the device while they load -------------------
 * No counterpart in the reference yet; its plan names safetensors as the weight source and on-load conversion as
 * the place where quantised encodings are produced (docs/plans/main-plan.md:26, :76, :112).
 * The file is read by the library during the call (header: 8-byte little-endian length + JSON; tensor data
 * follows); nothing of it is kept afterwards.  Source dtypes F32, F16 and BF16 are accepted.  F8_E4M3 / F8_E5M2
 * payloads and the "fnuz" flavours are rejected by name (ULLM_STATUS_UNSUPPORTED): an e4m3fn code must never be
 * read as e4m3fnuz or the other way round (docs/compatibility/amd-gpu.md:88-89). */
typedef struct ullm_cuda_safetensors_info_t {
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t dtype;       /* ULLM_CUDA_DTYPE_* of the stored tensor */
  uint32_t rank;        /* 1 or 2 (a rank-1 tensor is reported as [1, cols]) */
  uint64_t rows;
  uint64_t cols;
  uint64_t data_offset; /* of the tensor's first byte, from the start of the file */
  uint64_t data_bytes;
  uint32_t reserved[4];
} ullm_cuda_safetensors_info_t;
/* Header only: no device is touched.  ULLM_STATUS_INVALID_ARGUMENT for a file that is not safetensors or a name it
 * does not hold (the sink names what was wrong). */
ULLM_CUDA_API ullm_status_t ullm_cuda_safetensors_find(const char *path, const char *tensor_name,
                                         ullm_cuda_safetensors_info_t *info, ullm_cuda_error_sink_t *error_sink);
/* Reads tensor [N, K] in row chunks through the queue's pinned staging memory, converts to fp32 on the device and
 * quantises each chunk straight into weight.values / weight.scales (the same quantiser as ullm_cuda_quantize, so
 * the bytes equal quantising the fp32 tensor in one piece).  weight.n / weight.k must equal the stored shape.
 * Synchronous with respect to the caller like ullm_cuda_buffer_upload. */
ULLM_CUDA_API ullm_status_t ullm_cuda_quantize_safetensors(ullm_cuda_queue_t *queue, const char *path, const char *tensor_name,
                                             const ullm_cuda_weight_t *weight, ullm_cuda_error_sink_t *error_sink);

/* ---- the linear op: y[M,N] = prologue(x)[M,K] . W'[N,K]^T, fp32 accumulate ------ */
#define ULLM_CUDA_PROLOGUE_NONE UINT32_C(0)
#define ULLM_CUDA_PROLOGUE_RMSNORM UINT32_C(1) /* x <- bf16(x * rsqrt(mean(x^2) + eps) * gamma); gamma = 1 without norm_weight */
#define ULLM_CUDA_PROLOGUE_SWIGLU UINT32_C(2)  /* input is [M,2K] (gate | up); x <- bf16(silu(gate) * up) */

#define ULLM_CUDA_EPILOGUE_NONE UINT32_C(0)
/* Weight rows are [gate(N/2) | up(N/2)]; the output is [M, N/2]:
 * y[m][j] = bf16( silu(g) * u ),  g = bf16(x . W'[j]),  u = bf16(x . W'[N/2 + j]). */
#define ULLM_CUDA_EPILOGUE_SWIGLU UINT32_C(1)

#define ULLM_CUDA_KERNEL_AUTO UINT32_C(0)
#define ULLM_CUDA_KERNEL_MATVEC UINT32_C(1) /* CUDA-core streaming kernel, M <= 8; AUTO picks it for M = 1 (AQ4: M <= 4) */
#define ULLM_CUDA_KERNEL_GEMM UINT32_C(2)   /* tcgen05 / TMEM kernel */

typedef struct ullm_cuda_linear_desc_t {
  uint32_t struct_size;
  uint32_t abi_version;
  ullm_cuda_weight_t weight;
  uint64_t m;
  ullm_cuda_tensor_t input;
  uint64_t input_row_stride; /* elements; 0 = dense */
  ullm_cuda_tensor_t output;
  uint64_t output_row_stride; /* elements; 0 = dense (N, or N/2 with the SwiGLU epilogue) */
  uint32_t input_dtype;       /* BF16, or F32 (rounded to bf16 on load) */
  uint32_t output_dtype;      /* BF16 or F32 */
  uint32_t prologue;
  uint32_t kernel;
  float rms_eps;
  uint32_t epilogue;
  ullm_cuda_tensor_t norm_weight; /* RMSNorm prologue: gamma, bf16 [K]; buffer NULL = no weight vector */
  ullm_cuda_tensor_t residual;    /* f32 [M, N] added to the fp32 result before the output conversion
                                     (y = x . W'^T + residual; may alias the output); buffer NULL = none.
                                     Not offered together with the SwiGLU epilogue. */
  uint64_t residual_row_stride;   /* elements; 0 = dense (N) */
  uint32_t reserved[4];
} ullm_cuda_linear_desc_t;

/* Answers from the descriptor's shapes, dtypes and encoding alone: no handle is resolved and neither the
 * driver nor a device is touched.  OK, UNSUPPORTED (with a reason in the sink) or an argument error.
 * Mirrors Backend::supports (crates/ullm-core/src/backend.rs:8). */
ULLM_CUDA_API ullm_status_t ullm_cuda_linear_supports(const ullm_cuda_linear_desc_t *desc, uint32_t *selected_kernel,
                                        ullm_cuda_error_sink_t *error_sink);
/* Enqueue only (ordering by the queue; use ullm_cuda_queue_signal to observe completion).
 * Tensor-core (GEMM) linears stage their activations in scratch memory owned by the QUEUE, so linears on
 * different queues may overlap freely; the scratch grows on demand (not during a stream capture). */
ULLM_CUDA_API ullm_status_t ullm_cuda_linear_enqueue(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                       ullm_cuda_error_sink_t *error_sink);
/* Enqueue + signal in one call: the submit -> wait -> destroy shape of evidence_abi.h:48-59. */
ULLM_CUDA_API ullm_status_t ullm_cuda_linear_submit(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                      ullm_cuda_completion_t **completion,
                                      ullm_cuda_error_sink_t *error_sink);

/* No counterpart in the reference.  The same op as ullm_cuda_linear_enqueue on the tensor-core
 * (GEMM) kernel, for callers that must not trigger a device allocation: a serving loop that has
 * handed all free HBM to its own pool (so cudaMalloc would fail or fragment it), or a thread that
 * cannot afford the implicit device-wide synchronisation an allocation or a free may cause.
 * The GEMM path stages prologue(x) as two 8-bit planes plus one scale per token (M * K * 2 bytes and a
 * little more) before the tensor cores read it; here that staging area is a fixed
 * ULLM_CUDA_STATIC_SCRATCH_BYTES array compiled into the library (every GPU that loads the library
 * carries it until the process exits) instead of the queue's growable scratch.
 *   - M * K * 2 bytes must fit ULLM_CUDA_STATIC_SCRATCH_BYTES, else ULLM_STATUS_UNSUPPORTED;
 *     the SwiGLU epilogue is not offered here (ULLM_STATUS_UNSUPPORTED).
 *   - The first call on each device looks the array's device address up once; make that first
 *     call outside any stream capture.
 *   - All calls on a device share the one array and it keeps whatever the previous call left:
 *     nothing in it needs zeroing (each call overwrites exactly what it reads back), but two calls
 *     whose kernels can overlap on the GPU (different queues) race on it — serialise them.
 *   - No cudaMalloc / cudaFree / allocating library routine is called. */
#define ULLM_CUDA_STATIC_SCRATCH_BYTES (UINT64_C(8) << 20)
ULLM_CUDA_API ullm_status_t ullm_cuda_linear_enqueue_static_scratch(ullm_cuda_queue_t *queue,
                                                                    const ullm_cuda_linear_desc_t *desc,
                                                                    ullm_cuda_error_sink_t *error_sink);

/* ---- coarse command lists: prepare once, submit many times ---------------------------------------
 * The call unit the reference's runtime design fixes for its C ABI (docs/architecture/runtime.md:77-79): not one
 * call per kernel but a prepared plan of several ops.  PREPARE copies the reusable metadata (op kinds, shapes,
 * dtypes, encodings, prologues / epilogues) into storage the library owns and chooses every kernel, so that a
 * missing capability shows before anything runs; it keeps no pointer into the caller's arrays.  SUBMIT copies,
 * during the call, the resource bindings with the access mode each declares (AccessMode,
 * crates/ullm-core/src/handles.rs:12-16) and the dependency events, checks them against what each op needs, makes
 * the queue wait for the dependencies, enqueues all ops in order and returns a completion EVENT.  A synchronous
 * validation / enqueue failure is the status of submit itself; a failure after enqueue (a device-side wait that
 * gave up) is stored in the event, which owns its diagnostic (runtime.md:79), and read with event_query /
 * event_wait.  The context's executor owns every in-flight submission: destroying the event does not stop it from
 * being watched, and ullm_cuda_context_shutdown refuses new prepares / submits, drains what is in flight, and
 * collects the terminal statuses (runtime.md:63). */
#define ULLM_CUDA_ACCESS_READ UINT32_C(1) /* the values of ULLM_ACCESS_* (crates/ullm-hip-sys/src/bindings.rs:27-29) */
#define ULLM_CUDA_ACCESS_WRITE UINT32_C(2)
#define ULLM_CUDA_ACCESS_READ_WRITE UINT32_C(3)

#define ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT UINT32_C(1) /* the RMSNorm prologue takes a weight vector */
#define ULLM_CUDA_PLAN_OP_HAS_RESIDUAL UINT32_C(2)    /* a residual is added to the result */

typedef struct ullm_cuda_plan_op_t { /* one quantised linear of a plan: metadata only, no buffers */
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t encoding;
  uint32_t group_size;
  uint64_t n;
  uint64_t k;
  uint64_t m;
  uint32_t input_dtype;
  uint32_t output_dtype;
  uint32_t prologue;
  uint32_t epilogue;
  uint32_t kernel; /* ULLM_CUDA_KERNEL_AUTO or a forced kernel */
  uint32_t flags;  /* ULLM_CUDA_PLAN_OP_* */
  float rms_eps;
  uint32_t reserved[5];
} ullm_cuda_plan_op_t;

/* what a binding feeds */
#define ULLM_CUDA_SLOT_WEIGHT_VALUES UINT32_C(0)
#define ULLM_CUDA_SLOT_WEIGHT_SCALES UINT32_C(1)
#define ULLM_CUDA_SLOT_INPUT UINT32_C(2)
#define ULLM_CUDA_SLOT_OUTPUT UINT32_C(3)
#define ULLM_CUDA_SLOT_NORM_WEIGHT UINT32_C(4)
#define ULLM_CUDA_SLOT_RESIDUAL UINT32_C(5)

typedef struct ullm_cuda_binding_t {
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t op_index; /* which op of the plan */
  uint32_t slot;     /* ULLM_CUDA_SLOT_* */
  uint32_t access;   /* ULLM_CUDA_ACCESS_*: inputs must permit reading, the output writing; an output that
                        is also the op's residual must be READ_WRITE */
  uint32_t reserved0;
  ullm_cuda_tensor_t tensor;
  uint32_t reserved[4];
} ullm_cuda_binding_t;

/* Copies `count` op descriptions (1 .. 4096) and selects their kernels.  ULLM_STATUS_UNSUPPORTED names the first op
 * no kernel serves. */
ULLM_CUDA_API ullm_status_t ullm_cuda_prepare(ullm_cuda_context_t *context, const ullm_cuda_plan_op_t *ops, uint32_t count,
                                ullm_cuda_prepared_t **prepared, ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_prepared_destroy(ullm_cuda_prepared_t **prepared, ullm_cuda_error_sink_t *error_sink);
/* One submission of the whole plan on `queue`, after the `wait_count` events given (which may belong to other
 * queues of the context).  Every slot an op needs must be bound exactly once, with an access mode that permits
 * what the op does with it; an op must not write a span another binding of the same op reads, unless that is the
 * declared READ_WRITE output / residual pair.  `event` may be NULL when the caller will not observe completion. */
ULLM_CUDA_API ullm_status_t ullm_cuda_submit(ullm_cuda_queue_t *queue, ullm_cuda_prepared_t *prepared,
                               const ullm_cuda_binding_t *bindings, uint32_t binding_count,
                               ullm_cuda_event_t *const *wait_events, uint32_t wait_count, ullm_cuda_event_t **event,
                               ullm_cuda_error_sink_t *error_sink);
#define ULLM_CUDA_EVENT_PENDING UINT32_C(0)
#define ULLM_CUDA_EVENT_SUCCESS UINT32_C(1)
#define ULLM_CUDA_EVENT_FAILURE UINT32_C(2)
/* Never consumes the event.  state: pending, success, or failure (then the sink receives the stored diagnostic
 * and the return value is the stored status, e.g. ULLM_STATUS_CUDA_DEVICE_FLAGGED). */
ULLM_CUDA_API ullm_status_t ullm_cuda_event_query(ullm_cuda_event_t *event, uint32_t *state, ullm_cuda_error_sink_t *error_sink);
/* Polls up to timeout_ms (0 = one poll): OK on success, ULLM_STATUS_CUDA_TIMEOUT while pending, the stored status on failure. */
ULLM_CUDA_API ullm_status_t ullm_cuda_event_wait(ullm_cuda_event_t *event, uint32_t timeout_ms, ullm_cuda_error_sink_t *error_sink);
/* Drops the caller's reference; the executor keeps watching the submission until it completes or the context shuts down. */
ULLM_CUDA_API ullm_status_t ullm_cuda_event_destroy(ullm_cuda_event_t **event, ullm_cuda_error_sink_t *error_sink);
/* Closing state: new prepares and submits of this context are refused from now on; waits up to timeout_ms for every
 * in-flight submission (ULLM_STATUS_CUDA_TIMEOUT if some are still pending: call again); reports how many completed
 * with a failure.  The context can be destroyed afterwards like any other. */
ULLM_CUDA_API ullm_status_t ullm_cuda_context_shutdown(ullm_cuda_context_t *context, uint32_t timeout_ms, uint32_t *failed_submissions,
                                         ullm_cuda_error_sink_t *error_sink);

/* ---- the two halves of the fused all-reduce, as single ops --------------------------------------
 * No counterpart in the reference (it has no multi-GPU code).  The tensor-parallel stack below sums the partial
 * results of a row-parallel linear WITHOUT a collective kernel: the row-parallel linear stores every fp32
 * partial result together with a tag as one 8-byte {value, tag} pair into a slot per rank, and the linear that
 * follows adds the ranks' slots (plus an optional residual) while it stages its input, waiting — with the
 * context's wait limit — for any pair whose tag is not the expected one yet.  These two entries run the very
 * same kernels on slots inside an ordinary buffer of ONE device, so that a host can drive its own schedule
 * and so that the path can be checked without several GPUs (fill the slots of all "ranks" one launch after
 * the other, then gather).  Both serve 1 <= M <= 8 on the CUDA-core kernel only. */
typedef struct ullm_cuda_slots_t {
  uint32_t struct_size;
  uint32_t abi_version;
  ullm_cuda_tensor_t slots;   /* [ranks] slots of M * cols pairs {f32 value, u32 tag}, 16-byte aligned */
  uint64_t rank_stride_bytes; /* distance between two ranks' slots, a multiple of 16, >= M * cols * 8 */
  uint32_t ranks;             /* 1 .. 8 */
  uint32_t rank;              /* partial: the slot this launch fills; reduced: ignored */
  uint32_t tag;               /* written / expected with every value; any value, but a fresh one per use of the slots */
  uint32_t gather;            /* reduced: 0 = every thread block reads all slots, 1 = once per thread-block cluster */
  uint32_t reserved[4];
} ullm_cuda_slots_t;
/* y is not written: the fp32 results go to slot `rank` (cols = N).  No prologue restriction; no epilogue, no residual. */
ULLM_CUDA_API ullm_status_t ullm_cuda_linear_enqueue_partial(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                               const ullm_cuda_slots_t *slots, ullm_cuda_error_sink_t *error_sink);
/* x is not read: the input row m is bf16(desc->residual[m] + sum over ranks of slot[r][m]) (cols = K; here
 * desc->residual is [M, K] and belongs to the INPUT), then the prologue (NONE or RMSNORM), then the linear.
 * reduced_out, if its buffer is not NULL, receives the fp32 rows residual + sum (f32 [M, K], dense). */
ULLM_CUDA_API ullm_status_t ullm_cuda_linear_enqueue_reduced(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                               const ullm_cuda_slots_t *slots, ullm_cuda_tensor_t reduced_out,
                                               ullm_cuda_error_sink_t *error_sink);

/* ---- tensor-parallel communicator (NCCL, loaded at run time) ------------------- */
#define ULLM_CUDA_COMM_ID_BYTES 128
ULLM_CUDA_API ullm_status_t ullm_cuda_comm_unique_id(uint8_t id[ULLM_CUDA_COMM_ID_BYTES], ullm_cuda_error_sink_t *error_sink);
/* size up to 64 ranks; the fused all-reduce of the stack's decode path maps peer memory for up to 8 ranks of
 * one node and falls back to ncclAllReduce beyond that.  One stack at a time may use a communicator's peer
 * memory: a second live stack on the same communicator sums with ncclAllReduce. */
ULLM_CUDA_API ullm_status_t ullm_cuda_comm_create(ullm_cuda_context_t *context, const uint8_t id[ULLM_CUDA_COMM_ID_BYTES],
                                    uint32_t rank, uint32_t size, ullm_cuda_comm_t **comm,
                                    ullm_cuda_error_sink_t *error_sink);
/* in-place sum over ranks; dtype F32 or BF16 */
ULLM_CUDA_API ullm_status_t ullm_cuda_comm_all_reduce(ullm_cuda_comm_t *comm, ullm_cuda_queue_t *queue,
                                        ullm_cuda_tensor_t data, uint64_t count, uint32_t dtype,
                                        ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_comm_destroy(ullm_cuda_comm_t **comm, ullm_cuda_error_sink_t *error_sink);

/* ---- linear stack of a decoder: per layer QKV, O, gate+up, down; then the LM head, with the glue of a
 * decoder block around them (no attention is computed):
 *     h   = f32(input)
 *     qkv = QKV(rmsnorm(bf16 h, g1));   h += O(qkv[:, :q]);
 *     act = swiglu(GateUp(rmsnorm(bf16 h, g2)));   h += Down(act);     per layer
 *     logits = LMHead(rmsnorm(bf16 h, gf))
 * The residual stream h is fp32; the RMSNorm weight vectors are bf16(1 + z/8) from the seed.
 * Weights are generated on the device from the seed and quantised in place.
 * tp_size > 1: QKV, gate+up and the LM head are column-parallel (this rank holds
 * its slice of N), O and down are row-parallel (this rank holds its slice of K)
 * followed by a sum over ranks. ------------------------------------------------- */
typedef struct ullm_cuda_stack_desc_t {
  uint32_t struct_size;
  uint32_t abi_version;
  uint32_t encoding; /* AQ4 or FP8_CHANNEL */
  uint32_t layers;
  uint32_t hidden;
  uint32_t q_heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t ffn;
  uint32_t vocab;
  uint32_t tp_rank;
  uint32_t tp_size;
  uint32_t max_tokens; /* largest M of one step */
  uint32_t flags;
  uint64_t seed;
  float rms_eps;
  uint32_t reserved[5];
} ullm_cuda_stack_desc_t;

#define ULLM_CUDA_STACK_FLAG_NO_GRAPH UINT32_C(1) /* launch kernels directly instead of replaying a graph */
#define ULLM_CUDA_STACK_FLAG_KEEP_ACTIVATIONS UINT32_C(2) /* one activation set per layer, readable after a step */
#define ULLM_CUDA_STACK_FLAG_NCCL_ONLY UINT32_C(4) /* sum over ranks with ncclAllReduce even for decode steps */
/* How the kernel that follows a row-parallel linear gathers the ranks' partial sums (fused all-reduce, decode):
 * by default the blocks of a thread-block cluster share one reading of the ranks' slots through distributed shared
 * memory; the alternative is that every thread block reads all ranks' slots itself.  These two flags force one way. */
#define ULLM_CUDA_STACK_FLAG_GATHER_PER_BLOCK UINT32_C(8)
#define ULLM_CUDA_STACK_FLAG_GATHER_PER_CLUSTER UINT32_C(16)

ULLM_CUDA_API ullm_status_t ullm_cuda_stack_create(ullm_cuda_context_t *context, ullm_cuda_queue_t *queue,
                                     ullm_cuda_comm_t *comm, const ullm_cuda_stack_desc_t *desc,
                                     ullm_cuda_stack_t **stack, ullm_cuda_error_sink_t *error_sink);
/* One pass over all linears for m tokens: input bf16 [m,hidden] -> output bf16
 * [m, vocab/tp_size] (this rank's slice of the logits).  Enqueue only. */
ULLM_CUDA_API ullm_status_t ullm_cuda_stack_step(ullm_cuda_stack_t *stack, uint64_t m, ullm_cuda_tensor_t input_bf16,
                                   ullm_cuda_tensor_t output_bf16, ullm_cuda_error_sink_t *error_sink);
/* The same pass from and to HOST memory: pinned staging, host->device copy,
 * the step, device->host copy, and a bounded wait, all inside the call. */
ULLM_CUDA_API ullm_status_t ullm_cuda_stack_step_host(ullm_cuda_stack_t *stack, uint64_t m, const void *host_input_bf16,
                                        void *host_output_bf16, uint32_t timeout_ms,
                                        ullm_cuda_error_sink_t *error_sink);

#define ULLM_CUDA_STACK_LINEAR_QKV UINT32_C(0)
#define ULLM_CUDA_STACK_LINEAR_O UINT32_C(1)
#define ULLM_CUDA_STACK_LINEAR_GATE_UP UINT32_C(2)
#define ULLM_CUDA_STACK_LINEAR_DOWN UINT32_C(3)
#define ULLM_CUDA_STACK_LINEAR_LM_HEAD UINT32_C(4) /* layer index ignored */

typedef struct ullm_cuda_stack_linear_info_t {
  uint32_t struct_size;
  uint32_t abi_version;
  ullm_cuda_weight_t weight; /* this rank's shard */
  uint64_t tensor_id;        /* stream id of the full (unsharded) fp32 weight */
  uint64_t full_n;
  uint64_t full_k;
  uint64_t row_begin; /* shard origin inside the full weight */
  uint64_t col_begin;
  ullm_cuda_tensor_t last_input;  /* activation span this linear read in the last step */
  ullm_cuda_tensor_t last_output; /* and the span it wrote (row-parallel linears: residual + sum over ranks) */
  uint32_t input_dtype;
  uint32_t output_dtype;
  uint32_t prologue;
  uint32_t epilogue;
  ullm_cuda_tensor_t norm_weight;   /* gamma of the RMSNorm prologue, bf16 [K]; buffer NULL when there is none */
  ullm_cuda_tensor_t last_residual; /* f32 [m, N] added to the result in the last step; buffer NULL when none */
  uint64_t norm_tensor_id;          /* stream id of gamma */
  uint32_t reserved[4];
} ullm_cuda_stack_linear_info_t;

ULLM_CUDA_API ullm_status_t ullm_cuda_stack_linear_info(ullm_cuda_stack_t *stack, uint32_t layer, uint32_t which,
                                          ullm_cuda_stack_linear_info_t *info,
                                          ullm_cuda_error_sink_t *error_sink);
/* weight + scale bytes this rank streams per step, and kernels per step */
ULLM_CUDA_API ullm_status_t ullm_cuda_stack_stats(ullm_cuda_stack_t *stack, uint64_t *weight_bytes, uint64_t *launches_per_step,
                                    ullm_cuda_error_sink_t *error_sink);
ULLM_CUDA_API ullm_status_t ullm_cuda_stack_destroy(ullm_cuda_stack_t **stack, ullm_cuda_error_sink_t *error_sink);

#ifdef __cplusplus
} /* extern "C" */

#include <cstddef>
/* layout pins in the style of native/hip/src/evidence_abi.h:66-119 */
static_assert(sizeof(ullm_cuda_error_sink_t) == 48U, "error sink ABI layout changed");
static_assert(alignof(ullm_cuda_error_sink_t) == 8U, "error sink ABI alignment changed");
static_assert(offsetof(ullm_cuda_error_sink_t, message) == 8U, "error sink message offset changed");
static_assert(offsetof(ullm_cuda_error_sink_t, message_capacity) == 16U, "error sink capacity offset changed");
static_assert(offsetof(ullm_cuda_error_sink_t, message_length) == 24U, "error sink length offset changed");
static_assert(offsetof(ullm_cuda_error_sink_t, reserved) == 32U, "error sink reserved offset changed");
static_assert(sizeof(ullm_cuda_version_info_t) == 32U, "version info ABI layout changed");
static_assert(sizeof(ullm_cuda_backend_probe_result_t) == 64U, "backend probe ABI layout changed");
static_assert(sizeof(ullm_cuda_context_probe_result_t) == 32U, "context probe ABI layout changed");
static_assert(sizeof(ullm_cuda_tensor_t) == 16U, "tensor span ABI layout changed");
static_assert(sizeof(ullm_cuda_weight_t) == 56U, "weight ABI layout changed");
static_assert(sizeof(ullm_cuda_completion_result_t) == 56U, "completion result ABI layout changed");
static_assert(sizeof(ullm_cuda_linear_desc_t) == 200U, "linear descriptor ABI layout changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, norm_weight) == 144U, "linear norm_weight offset changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, residual) == 160U, "linear residual offset changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, weight) == 8U, "linear weight offset changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, m) == 64U, "linear m offset changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, input) == 72U, "linear input offset changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, output) == 96U, "linear output offset changed");
static_assert(offsetof(ullm_cuda_linear_desc_t, input_dtype) == 120U, "linear input_dtype offset changed");
static_assert(sizeof(ullm_cuda_slots_t) == 64U, "slots descriptor ABI layout changed");
static_assert(sizeof(ullm_cuda_plan_op_t) == 88U, "plan op ABI layout changed");
static_assert(sizeof(ullm_cuda_safetensors_info_t) == 64U, "safetensors info ABI layout changed");
static_assert(sizeof(ullm_cuda_binding_t) == 56U, "binding ABI layout changed");
static_assert(sizeof(ullm_cuda_stack_desc_t) == 88U, "stack descriptor ABI layout changed");
static_assert(sizeof(ullm_cuda_stack_linear_info_t) == 208U, "stack linear info ABI layout changed");
#endif

#endif /* ULLM_CUDA_H */

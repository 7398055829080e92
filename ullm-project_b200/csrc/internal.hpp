// Shared internals of libullm_cuda: boundary helpers (error sink, versioned-struct
// validation, handle registries) and the runtime objects behind the opaque handles.
//
// Boundary rules implemented here follow the reference's host stub:
//   sink validation without writing a message   native/hip/src/hip_stub.cpp:43-66
//   write_error truncation / BUFFER_TOO_SMALL   native/hip/src/hip_stub.cpp:17-41
//   struct_size / abi_version / reserved checks native/hip/src/hip_stub.cpp:69-118
#pragma once

#include "ullm_cuda.h"

#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <mutex>
#include <string>
#include <unordered_set>
#include <vector>

namespace ullm {

using sink_t = ullm_cuda_error_sink_t;

// ---- error sink -----------------------------------------------------------

inline ullm_status_t write_error(sink_t *sink, ullm_status_t primary, const char *message) noexcept {
  if (sink == nullptr) return primary;
  const size_t len = message == nullptr ? 0U : std::strlen(message);
  sink->message_length = static_cast<uint64_t>(len);
  if (sink->message_capacity == 0U) return ULLM_STATUS_BUFFER_TOO_SMALL;
  if (sink->message == nullptr) return ULLM_STATUS_INVALID_ARGUMENT;
  const size_t cap = static_cast<size_t>(sink->message_capacity);
  const size_t n = len < cap - 1U ? len : cap - 1U;
  if (n != 0U) std::memcpy(sink->message, message, n);
  sink->message[n] = '\0';
  return len <= cap - 1U ? primary : ULLM_STATUS_BUFFER_TOO_SMALL;
}

inline ullm_status_t errorf(sink_t *sink, ullm_status_t primary, const char *fmt, ...) noexcept {
  char text[512];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(text, sizeof(text), fmt, ap);
  va_end(ap);
  return write_error(sink, primary, text);
}

inline ullm_status_t validate_sink(sink_t *sink) noexcept {
  if (sink == nullptr) return ULLM_STATUS_OK;
  if (sink->struct_size < sizeof(sink_t)) return ULLM_STATUS_INVALID_ARGUMENT;
  if (sink->abi_version != ULLM_CUDA_ABI_VERSION) return ULLM_STATUS_INVALID_ABI_VERSION;
  if (sink->reserved[0] != 0U || sink->reserved[1] != 0U) return ULLM_STATUS_RESERVED_NONZERO;
  if (sink->message_capacity > static_cast<uint64_t>(std::numeric_limits<size_t>::max()))
    return ULLM_STATUS_INVALID_ARGUMENT;
  if (sink->message_capacity != 0U && sink->message == nullptr) return ULLM_STATUS_INVALID_ARGUMENT;
  sink->message_length = 0U;
  if (sink->message != nullptr && sink->message_capacity != 0U) sink->message[0] = '\0';
  return ULLM_STATUS_OK;
}

// struct_size / abi_version / reserved, in that order
template <typename S>
inline ullm_status_t validate_struct(const S *value, sink_t *sink, const char *what) noexcept {
  if (value == nullptr) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s is null", what);
  if (value->struct_size < sizeof(S))
    return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: struct_size is smaller than the ABI v1 struct", what);
  if (value->abi_version != ULLM_CUDA_ABI_VERSION)
    return errorf(sink, ULLM_STATUS_INVALID_ABI_VERSION, "%s: unsupported ABI version", what);
  for (size_t i = 0; i < sizeof(value->reserved) / sizeof(value->reserved[0]); ++i)
    if (value->reserved[i] != 0U)
      return errorf(sink, ULLM_STATUS_RESERVED_NONZERO, "%s: reserved fields must be zero", what);
  return ULLM_STATUS_OK;
}

// ---- runtime objects --------------------------------------------------------

constexpr uint32_t kMagicContext = 0x63747831U, kMagicQueue = 0x71756531U, kMagicBuffer = 0x62756631U,
                   kMagicCompletion = 0x636d7031U, kMagicGraph = 0x67726131U, kMagicComm = 0x636f6d31U,
                   kMagicStack = 0x73746b31U;

constexpr int kMaxDevices = 64;
constexpr uint32_t kDefaultWaitLimitMs = 20000;

struct Queue;
struct Submission;

struct Context {
  uint32_t magic = kMagicContext;
  int device = 0;
  int sm_count = 0;
  size_t l2_bytes = 0;
  size_t smem_optin = 0;
  uint32_t *host_flags = nullptr;    // [16] words, mapped pinned memory
  uint32_t *device_flags = nullptr;  // device view of host_flags: kernels set a word when a bounded wait expires
  // Device-resident abort word: set (with the flag word) by the first wait that gives up, read by every
  // later wait before it starts polling, so that all the work queued behind an expired wait unwinds in
  // about one limit instead of one limit per wait.  Cleared by the completion wait that reports it.
  uint32_t *abort_word = nullptr;
  std::atomic<uint32_t> wait_limit_ms{kDefaultWaitLimitMs};  // limit of every device-side wait
  std::mutex mutex;
  std::vector<cudaEvent_t> event_pool;
  std::vector<Queue *> queues;  // live queues (guarded by mutex): buffer_free checks that they are idle
  std::atomic<uint64_t> live_children{0};
  // the executor of the command-list path: every submission in flight, watched until it completes
  std::atomic<bool> closing{false};
  std::vector<Submission *> in_flight;  // guarded by mutex
};

// Device scratch of the GEMM path (activation planes, token scales, gate|up pairs, split-K partials and the
// split-K arrival counters).  One per queue: linears enqueued on different queues may overlap on the GPU, so
// they must not share staging memory or counters.
struct GemmScratch {
  void *ptr = nullptr;
  size_t bytes = 0;
  uint32_t *tile_counters = nullptr;  // zero between launches
  std::mutex mutex;
};

struct Queue {
  uint32_t magic = kMagicQueue;
  Context *ctx = nullptr;
  cudaStream_t stream = nullptr;
  std::mutex mutex;
  uint64_t dispatch_count = 0;  // kernels launched since the last signal
  uint64_t copy_count = 0;
  uint64_t total_dispatch = 0;
  bool capturing = false;
  void *staging = nullptr;  // pinned, kStagingBytes
  GemmScratch scratch;
};
constexpr size_t kStagingBytes = size_t(16) << 20;

struct Buffer {
  uint32_t magic = kMagicBuffer;
  Context *ctx = nullptr;
  void *ptr = nullptr;
  uint64_t size = 0;
};

struct Completion {
  uint32_t magic = kMagicCompletion;
  Queue *queue = nullptr;  // may have been destroyed since: check the registry before use
  Context *ctx = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t event = nullptr;
  uint64_t dispatch_count = 0;
  uint64_t copy_count = 0;
};

struct Graph {
  uint32_t magic = kMagicGraph;
  Context *ctx = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t kernel_nodes = 0;
};

// Live-handle registry: a stale, foreign or double-freed handle is answered
// with ULLM_STATUS_CUDA_INVALID_HANDLE instead of being dereferenced.
class Registry {
 public:
  void add(const void *p) {
    std::lock_guard<std::mutex> g(m_);
    live_.insert(p);
  }
  bool remove(const void *p) {
    std::lock_guard<std::mutex> g(m_);
    return live_.erase(p) != 0;
  }
  bool contains(const void *p) {
    std::lock_guard<std::mutex> g(m_);
    return p != nullptr && live_.count(p) != 0;
  }

 private:
  std::mutex m_;
  std::unordered_set<const void *> live_;
};
Registry &registry();

template <typename T>
inline T *checked(const void *handle) {
  return registry().contains(handle) ? const_cast<T *>(static_cast<const T *>(handle)) : nullptr;
}
inline Context *as_context(const ullm_cuda_context_t *h) {
  Context *c = checked<Context>(h);
  return (c && c->magic == kMagicContext) ? c : nullptr;
}
inline Queue *as_queue(const ullm_cuda_queue_t *h) {
  Queue *q = checked<Queue>(h);
  return (q && q->magic == kMagicQueue) ? q : nullptr;
}
inline Buffer *as_buffer(const ullm_cuda_buffer_t *h) {
  Buffer *b = checked<Buffer>(h);
  return (b && b->magic == kMagicBuffer) ? b : nullptr;
}

// ---- helpers used by every op ------------------------------------------------

ullm_status_t cuda_error(sink_t *sink, cudaError_t e, const char *what) noexcept;

#define ULLM_CUDA_TRY(expr, what)                                     \
  do {                                                                \
    cudaError_t ullm_e_ = (expr);                                     \
    if (ullm_e_ != cudaSuccess) return cuda_error(sink, ullm_e_, what); \
  } while (0)

// Resolves a span to a device pointer after checking handle, context, alignment and bounds.
ullm_status_t resolve(const ullm_cuda_tensor_t &t, uint64_t bytes, uint64_t align, const Context *ctx,
                      const char *what, sink_t *sink, void **out) noexcept;

// Queue acquisition for an op: valid handle, right device made current.
ullm_status_t begin_op(ullm_cuda_queue_t *queue, sink_t *sink, Queue **out) noexcept;
// false (with *status set) while resources wait too long to be retired: new work is refused.
bool submissions_open(sink_t *sink, ullm_status_t *status) noexcept;
// Runs `release` now if `stream` is observed idle, else in the background once a fence behind the
// stream's current work is reached.  Never blocks.  false = nothing can watch the fence (abandoned).
bool retire_behind(int device, cudaStream_t stream, std::function<void()> release) noexcept;
// Post-launch check + accounting.
ullm_status_t end_launch(Queue *q, sink_t *sink, const char *what, uint64_t kernels = 1) noexcept;

// Weight span checks shared by quantise / dequantise / linear.
struct WeightPtrs {
  const uint8_t *values = nullptr;
  const void *scales = nullptr;
  uint64_t n = 0, k = 0;
  uint32_t encoding = 0;
};
ullm_status_t resolve_weight(const ullm_cuda_weight_t &w, const Context *ctx, sink_t *sink,
                             WeightPtrs *out) noexcept;

inline uint64_t dtype_bytes(uint32_t dtype) {
  switch (dtype) {
    case ULLM_CUDA_DTYPE_BF16:
    case ULLM_CUDA_DTYPE_F16: return 2;
    case ULLM_CUDA_DTYPE_F32: return 4;
    case ULLM_CUDA_DTYPE_F8E4M3FN:
    case ULLM_CUDA_DTYPE_I8:
    case ULLM_CUDA_DTYPE_U8: return 1;
    default: return 0;
  }
}

// ---- fused all-reduce over peer memory (decode path) -------------------------------------------
// A row-parallel matvec writes every fp32 partial output together with a 32-bit tag as ONE 8-byte
// store into a slot of EVERY rank's symmetric buffer (plain peer stores over NVLink; 8-byte stores
// are single-copy atomic, so a reader that sees the tag sees the value: no fence, no flag word, no
// atomic).  The next kernel on each rank sums the ranks' slots while it stages its activations,
// re-reading (time-bounded) any pair whose tag is not yet the expected one: either every CTA reads
// all ranks' slots itself, or (cluster launch) each CTA of a thread-block cluster sums a share and
// hands it to the others through distributed shared memory, so that the slots are read once per
// cluster.  The tag is step_counter * uses_per_step + use + 1, where a one-thread kernel bumps
// step_counter once per step; two slot sets alternate per use of a site so that a fast rank never
// overwrites what a slow rank is still reading.
// Tag arithmetic is modulo 2^32.  A slot is rewritten every second use of its site, so the tag found in
// it is always the expected one or the one from two uses earlier; the two can only coincide 2^32 uses
// apart, and by the first wrap no slot still holds its initial zero.  Wrap-around is therefore harmless.
constexpr int kMaxPeers = 8;
struct PushOut {       // producer side
  uint8_t *peer_base[kMaxPeers];  // every rank's symmetric buffer as mapped here
  uint64_t slot_off[2];           // slot sets (pairs of {value, tag}), chosen by use parity
  uint64_t slot_stride;           // bytes between two ranks' slots
  const uint32_t *step_counter;   // local
  uint32_t uses_per_step, use;    // this site's position in the step's sequence of uses
  uint32_t tp = 0, rank = 0;      // tp == 0: disabled
};
struct PushIn {        // consumer side
  const uint8_t *local_base;
  uint64_t slot_off[2];
  uint64_t slot_stride;
  const uint32_t *step_counter;
  uint32_t uses_per_step, use;
  const float *residual;          // optional f32 [M, K]: the staged input is residual + sum over ranks
  float *reduced_out;             // optional f32 [M, K]: one thread block (or cluster) also stores that input here
  uint32_t tp = 0;
  uint32_t cluster = 0;           // 0: every thread block reads all ranks' slots; else blocks per cluster sharing one reading
};

// ---- internal launchers (raw device pointers; arguments already validated) -----

struct LinearArgs {
  const void *x = nullptr;   // bf16 or f32 [M, x_stride]
  void *y = nullptr;         // bf16 or f32 [M, y_stride]
  const uint8_t *w = nullptr;
  const void *scales = nullptr;
  uint32_t m = 0;
  uint32_t n = 0, k = 0;
  uint64_t x_stride = 0, y_stride = 0;
  uint32_t encoding = 0;
  uint32_t x_dtype = 0, y_dtype = 0;
  uint32_t prologue = 0;
  uint32_t epilogue = 0;
  float rms_eps = 1e-5f;
  const void *norm_weight = nullptr;  // RMSNorm prologue: bf16 gamma[K], or null
  const float *residual = nullptr;    // f32 [M, res_stride]: y = x . W'^T + residual (may alias y)
  uint64_t res_stride = 0;
  uint32_t wait_limit_ms = kDefaultWaitLimitMs;  // limit of the kernel's device-side waits
  uint32_t *abort_word = nullptr;                // the context's device-resident abort word
  PushOut push_out{};  // matvec only: write the fp32 output into every rank's slot instead of y
  PushIn push_in{};    // matvec only: the input is the sum of the ranks' slots
};

// returns the number of kernels launched, or -1 after setting *err
int launch_matvec(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err);
// NVFP4 (nvfp4.cu): its own decode kernel, quantiser and dequantiser
bool nvfp4_matvec_supports(const LinearArgs &a, const char **why);
int launch_matvec_nvfp4(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err);
uint64_t nvfp4_scale_bytes(uint64_t n, uint64_t k);
void launch_nvfp4_quantize(cudaStream_t s, const float *src, uint64_t n, uint64_t k, uint8_t *values, void *scales);
void launch_nvfp4_dequantize(cudaStream_t s, const uint8_t *values, const void *scales, uint64_t n, uint64_t k, void *out,
                             uint32_t out_dtype);
bool matvec_supports(const LinearArgs &a, const char **why);

// `scratch` is the staging memory of the queue whose stream is given (grown on demand, not during capture).
int launch_gemm(const Context *ctx, GemmScratch *scratch, cudaStream_t stream, const LinearArgs &a, cudaError_t *err);
// The GEMM path with its activation staging area in a fixed file-scope device array (no allocation).
// Returns kernels launched, -1 with *err set, or -2 when the arguments do not fit the array.
int launch_gemm_static_scratch(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err);
// Scratch bytes launch_gemm needs for these arguments, and a way to reserve them ahead of
// time (the scratch may not grow while a stream is being captured).
size_t gemm_scratch_bytes(const Context *ctx, const LinearArgs &a);
cudaError_t gemm_reserve_scratch(GemmScratch *scratch, size_t bytes);
// Shape-only answer (no device, no driver): `a.w` may be null.
bool gemm_supports(const LinearArgs &a, const char **why);
// Kernel behind ULLM_CUDA_KERNEL_AUTO when both serve the shape.  Measured on weights larger than L2: the
// tensor-core path streams FP8 weights faster than the CUDA-core matvec from two tokens on (5.2 vs 3.7 TB/s
// at M=2, 2.7 vs 0.84 at M=8); for AQ4 it wins from five tokens on (1.6 vs 1.0 TB/s at M=8, 1.6 vs 1.9 at M=4).
inline bool auto_prefers_gemm(const LinearArgs &a) {
  return a.encoding == ULLM_CUDA_ENCODING_FP8_CHANNEL ? a.m >= 2 : a.m >= 5;
}

void launch_synth_weights(cudaStream_t s, uint64_t seed, uint64_t tensor_id, uint64_t first, uint64_t count,
                          float std, float *out);
void launch_synth_activations(cudaStream_t s, uint64_t seed, uint64_t tensor_id, uint64_t first, uint64_t count,
                              void *out_bf16);
// Strided variant used by the stack: rows [row0,row0+n) x cols [col0,col0+k) of a [*, full_k] tensor.
void launch_synth_weight_tile(cudaStream_t s, uint64_t seed, uint64_t tensor_id, uint64_t full_k, uint64_t row0,
                              uint64_t col0, uint64_t n, uint64_t k, float std, float *out);
void launch_quantize(cudaStream_t s, const float *src, uint32_t encoding, uint64_t n, uint64_t k, uint8_t *values,
                     void *scales);
void launch_aq4_unpack(cudaStream_t s, const uint8_t *values, uint64_t bytes, int8_t *out);
void launch_aq4_pack(cudaStream_t s, const int8_t *src, uint64_t bytes, uint8_t *values);
void launch_dequantize(cudaStream_t s, uint32_t encoding, const uint8_t *values, const void *scales, uint64_t n,
                       uint64_t k, void *out, uint32_t out_dtype);

// ---- the linear op's shared entry points (linear.cu), used by the command-list path (plan.cu)
ullm_status_t enqueue_linear_desc(Queue *q, const ullm_cuda_linear_desc_t *desc, sink_t *sink);
ullm_status_t linear_shape_check(const ullm_cuda_linear_desc_t *desc, uint32_t *kernel, sink_t *sink);
// Reads and clears the context's device-side failure words; non-zero = some kernel gave up a bounded wait.
// Re-arms the device-resident abort word behind `stream` (or at once when it is null).
uint32_t take_device_flags(Context *ctx, cudaStream_t stream, uint32_t (&words)[4]);

// comm internals used by the stack
struct Comm;
// Collective: every rank calls it with the same size.  true = this rank's zeroed symmetric buffer of at least
// `bytes` is mapped on every rank and reserved for the caller until comm_sym_release; false = not available
// (no peer access, or another user holds it): the same verdict on every rank.
bool comm_sym_setup(Comm *c, size_t bytes, std::string *why);
void comm_sym_release(Comm *c);
bool comm_p2p(const Comm *c);
uint8_t *comm_sym_ptr(const Comm *c, uint32_t peer);
size_t comm_sym_bytes(const Comm *c);
Comm *as_comm(const ullm_cuda_comm_t *h);
cudaError_t comm_all_reduce_raw(Comm *c, cudaStream_t s, void *data, uint64_t count, uint32_t dtype,
                                std::string *why);
uint32_t comm_size(const Comm *c);
uint32_t comm_rank(const Comm *c);

}  // namespace ullm

#define ULLM_ENTRY_BEGIN try {
#define ULLM_ENTRY_END(name)                                                                              \
  }                                                                                                       \
  catch (...) {                                                                                           \
    return ullm::write_error(error_sink, ULLM_STATUS_INTERNAL_ERROR, "unexpected exception in " name);    \
  }

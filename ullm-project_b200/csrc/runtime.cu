// Context / queue / buffer / completion / graph objects and the version and probe
// entry points of libullm_cuda.
//
// Lifecycle follows the reference's HIP evidence runtime, re-expressed so that
// nothing is allocated per request:
//   stream + event + device buffers per request   native/hip/src/hip_evidence_runtime.hip.cpp:53-71, :585-659
//   poll-with-deadline wait, timeout 0 = one poll  native/hip/src/hip_evidence_runtime.hip.cpp:508-535
//   consume-once completion handles               native/hip/src/hip_evidence_runtime.hip.cpp:691-698
//   exact-architecture check before any work      native/hip/src/hip_evidence_runtime.hip.cpp:463-496
//   never free what is not proven complete; a background reaper with a bounded number of slots retires
//   such resources, and new submissions are refused once a retirement stays unproven
//                                                 native/hip/src/hip_evidence_runtime.hip.cpp:77-103, :151-257
// There is no CPU fallback: without a usable sm_100 device every compute entry
// answers ULLM_STATUS_CUDA_UNAVAILABLE (native/hip/src/hip_evidence_stub.cpp:103-127).
#include "internal.hpp"

#include <chrono>
#include <condition_variable>
#include <memory>
#include <new>
#include <thread>

namespace ullm {

Registry &registry() {
  static Registry *r = new Registry();  // leaked on purpose: handles may outlive static destruction
  return *r;
}

ullm_status_t cuda_error(sink_t *sink, cudaError_t e, const char *what) noexcept {
  ullm_status_t st = ULLM_STATUS_CUDA_RUNTIME_ERROR;
  if (e == cudaErrorMemoryAllocation) st = ULLM_STATUS_CUDA_OUT_OF_MEMORY;
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInitializationError ||
      e == cudaErrorNotSupported)
    st = ULLM_STATUS_CUDA_UNAVAILABLE;
  return errorf(sink, st, "%s: %s (%s); no CPU fallback exists", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// The library is compiled for sm_100a only; any other device is "unavailable",
// never silently served by different code.
static bool device_is_target(int device, cudaDeviceProp *prop_out, cudaError_t *err) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (err) *err = e;
  if (e != cudaSuccess) return false;
  if (prop_out) *prop_out = prop;
  return prop.major == 10 && prop.minor == 0;
}

ullm_status_t resolve(const ullm_cuda_tensor_t &t, uint64_t bytes, uint64_t align, const Context *ctx,
                      const char *what, sink_t *sink, void **out) noexcept {
  Buffer *b = as_buffer(t.buffer);
  if (b == nullptr) return errorf(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "%s: buffer handle is not live", what);
  if (ctx != nullptr && b->ctx != ctx)
    return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: buffer belongs to another context", what);
  if (align > 1 && (t.offset_bytes % align) != 0)
    return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: offset %llu is not %llu-byte aligned", what,
                  (unsigned long long)t.offset_bytes, (unsigned long long)align);
  if (t.offset_bytes > b->size || bytes > b->size - t.offset_bytes)
    return errorf(sink, ULLM_STATUS_CUDA_OUT_OF_RANGE, "%s: span [%llu, +%llu) leaves a %llu-byte buffer", what,
                  (unsigned long long)t.offset_bytes, (unsigned long long)bytes, (unsigned long long)b->size);
  *out = static_cast<uint8_t *>(b->ptr) + t.offset_bytes;
  return ULLM_STATUS_OK;
}

ullm_status_t begin_op(ullm_cuda_queue_t *queue, sink_t *sink, Queue **out) noexcept {
  Queue *q = as_queue(queue);
  if (q == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "queue handle is not live");
  ULLM_CUDA_TRY(cudaSetDevice(q->ctx->device), "cudaSetDevice");
  *out = q;
  return ULLM_STATUS_OK;
}

ullm_status_t end_launch(Queue *q, sink_t *sink, const char *what, uint64_t kernels) noexcept {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_error(sink, e, what);
  std::lock_guard<std::mutex> g(q->mutex);
  q->dispatch_count += kernels;
  q->total_dispatch += kernels;
  return ULLM_STATUS_OK;
}

ullm_status_t resolve_weight(const ullm_cuda_weight_t &w, const Context *ctx, sink_t *sink,
                             WeightPtrs *out) noexcept {
  if (w.encoding != ULLM_CUDA_ENCODING_AQ4 && w.encoding != ULLM_CUDA_ENCODING_FP8_CHANNEL && w.encoding != ULLM_CUDA_ENCODING_NVFP4)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "weight encoding must be AQ4, FP8_CHANNEL or NVFP4");
  if (w.n == 0 || w.k == 0) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight has a zero extent");
  if (w.n > 0x7fffffffULL || w.k > 0x7fffffffULL)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "weight extents above 2^31-1 are not supported");
  uint64_t vbytes, sbytes;
  if (w.encoding == ULLM_CUDA_ENCODING_NVFP4) {
    if (w.group_size != ULLM_CUDA_NVFP4_BLOCK)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "NVFP4 block size must be 16");
    if (w.k % 32 != 0)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "NVFP4 needs K to be a multiple of 32; ragged K is rejected");
    vbytes = w.n * (w.k / 2);
    sbytes = nvfp4_scale_bytes(w.n, w.k);
  } else if (w.encoding == ULLM_CUDA_ENCODING_AQ4) {
    if (w.group_size != ULLM_CUDA_AQ4_GROUP)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "AQ4 group size must be 128");
    if (w.k % ULLM_CUDA_AQ4_GROUP != 0)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "AQ4 needs K to be a multiple of 128; ragged K is rejected");
    vbytes = w.n * (w.k / 2);
    sbytes = w.n * (w.k / ULLM_CUDA_AQ4_GROUP) * 2;
  } else {
    if (w.group_size != 0)
      return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "FP8_CHANNEL takes group_size 0");
    if (w.k % 16 != 0)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "FP8_CHANNEL needs K to be a multiple of 16");
    vbytes = w.n * w.k;
    sbytes = w.n * 4;
  }
  void *v = nullptr, *s = nullptr;
  ullm_status_t st = resolve(w.values, vbytes, 16, ctx, "weight values", sink, &v);
  if (st != ULLM_STATUS_OK) return st;
  st = resolve(w.scales, sbytes, w.encoding == ULLM_CUDA_ENCODING_NVFP4 ? 16 : 4, ctx, "weight scales", sink, &s);
  if (st != ULLM_STATUS_OK) return st;
  out->values = static_cast<const uint8_t *>(v);
  out->scales = s;
  out->n = w.n;
  out->k = w.k;
  out->encoding = w.encoding;
  return ULLM_STATUS_OK;
}


// ---- retirement of resources whose completion is not yet proven ---------------------------------
// A destructor never blocks on the device.  When the work that may still use a resource has not been
// observed complete (cudaEventQuery / cudaStreamQuery), the resource is handed, together with a fence
// event, to a background thread that polls the fence and releases the resource once it is reached.  A
// fence that is not reached within kRetireDeadline is abandoned: the resource is leaked on purpose (the
// process exit reclaims it) and the breaker opens, after which submissions are refused.  The number of
// pending retirements is bounded; beyond it submissions are refused until the reaper catches up.
namespace {

constexpr size_t kMaxRetireSlots = 8;
constexpr auto kRetireDeadline = std::chrono::seconds(120);

struct Retired {
  int device = 0;
  cudaEvent_t fence = nullptr;            // recorded behind the last use
  std::function<void()> release;          // frees the resources; runs with `device` current
  std::chrono::steady_clock::time_point deadline;
  Retired *next = nullptr;
};

class Reaper {
 public:
  bool start() noexcept {
    std::lock_guard<std::mutex> g(m_);
    if (started_) return true;
    try {
      std::thread(&Reaper::run, this).detach();  // never joined: process exit must not wait for the device
      started_ = true;
    } catch (...) {
      started_ = false;
    }
    return started_;
  }
  // false: the breaker is open or every slot is taken
  bool accepting() noexcept {
    std::lock_guard<std::mutex> g(m_);
    return !blocked_ && pending_ < kMaxRetireSlots;
  }
  bool blocked() noexcept {
    std::lock_guard<std::mutex> g(m_);
    return blocked_;
  }
  size_t pending() noexcept {
    std::lock_guard<std::mutex> g(m_);
    return pending_;
  }
  void enqueue(Retired *r) noexcept {
    std::lock_guard<std::mutex> g(m_);
    r->next = nullptr;
    if (tail_ == nullptr) head_ = r; else tail_->next = r;
    tail_ = r;
    ++pending_;
    cv_.notify_one();
  }

 private:
  void run() noexcept {
    for (;;) {
      Retired *r = nullptr;
      {
        std::unique_lock<std::mutex> lk(m_);
        cv_.wait(lk, [this] { return head_ != nullptr; });
        r = head_;
        head_ = r->next;
        if (head_ == nullptr) tail_ = nullptr;
      }
      bool proven = false;
      (void)cudaSetDevice(r->device);
      for (;;) {
        const cudaError_t e = cudaEventQuery(r->fence);
        if (e == cudaSuccess) {
          proven = true;
          break;
        }
        if (e != cudaErrorNotReady) {
          (void)cudaGetLastError();
          break;  // the runtime is unhealthy: nothing is proven
        }
        if (std::chrono::steady_clock::now() >= r->deadline) break;
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      if (proven) {
        try {
          r->release();
        } catch (...) {
        }
        (void)cudaEventDestroy(r->fence);
        delete r;
        std::lock_guard<std::mutex> g(m_);
        --pending_;
      } else {
        // leaked on purpose: safety before reclamation
        std::lock_guard<std::mutex> g(m_);
        blocked_ = true;
      }
    }
  }
  std::mutex m_;
  std::condition_variable cv_;
  Retired *head_ = nullptr, *tail_ = nullptr;
  size_t pending_ = 0;
  bool started_ = false, blocked_ = false;
};

Reaper &reaper() {
  static Reaper *r = new Reaper();  // leaked on purpose, like the registry
  return *r;
}

}  // namespace

uint32_t take_device_flags(Context *ctx, cudaStream_t stream, uint32_t (&words)[4]) {
  uint32_t any = 0;
  std::lock_guard<std::mutex> g(ctx->mutex);
  for (int i = 0; i < 16; ++i) {
    const uint32_t w = const_cast<volatile uint32_t *>(ctx->host_flags)[i];
    if (i < 4) words[i] = w;
    any |= w;
  }
  if (any != 0U) {
    for (int i = 0; i < 16; ++i) const_cast<volatile uint32_t *>(ctx->host_flags)[i] = 0U;
    if (stream != nullptr)
      (void)cudaMemsetAsync(ctx->abort_word, 0, sizeof(uint32_t), stream);
    else
      (void)cudaMemset(ctx->abort_word, 0, sizeof(uint32_t));
  }
  return any;
}

bool submissions_open(sink_t *sink, ullm_status_t *status) noexcept {
  if (reaper().accepting()) return true;
  *status = write_error(sink, ULLM_STATUS_CUDA_RUNTIME_ERROR,
                        reaper().blocked() ? "an earlier retirement could not be proven complete; new submissions are refused"
                                           : "too many resources are waiting to be retired; try again later");
  return false;
}

// Releases `release` now when `stream` is observed idle, otherwise behind a fence on it.  Never blocks.
// Returns false when the resources had to be abandoned (no fence could be made).
bool retire_behind(int device, cudaStream_t stream, std::function<void()> release) noexcept {
  (void)cudaSetDevice(device);
  const cudaError_t q = cudaStreamQuery(stream);
  if (q == cudaSuccess) {
    release();
    return true;
  }
  (void)cudaGetLastError();
  Retired *r = new (std::nothrow) Retired();
  cudaEvent_t ev = nullptr;
  if (r == nullptr || !reaper().start() || cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventRecord(ev, stream) != cudaSuccess) {
    (void)cudaGetLastError();
    if (ev != nullptr) (void)cudaEventDestroy(ev);
    delete r;
    return false;  // leaked: completion cannot be proven and nothing can watch for it
  }
  r->device = device;
  r->fence = ev;
  r->release = std::move(release);
  r->deadline = std::chrono::steady_clock::now() + kRetireDeadline;
  reaper().enqueue(r);
  return true;
}

static cudaEvent_t take_event(Context *ctx, cudaError_t *err) {
  {
    std::lock_guard<std::mutex> g(ctx->mutex);
    if (!ctx->event_pool.empty()) {
      cudaEvent_t e = ctx->event_pool.back();
      ctx->event_pool.pop_back();
      *err = cudaSuccess;
      return e;
    }
  }
  cudaEvent_t e = nullptr;
  *err = cudaEventCreate(&e);
  return e;
}

static void give_event(Context *ctx, cudaEvent_t e) {
  std::lock_guard<std::mutex> g(ctx->mutex);
  ctx->event_pool.push_back(e);
}

// Polls with a deadline; never blocks without one.  Spins briefly before it
// starts sleeping so that microsecond-scale work is not rounded up to a sleep.
static cudaError_t poll_event(cudaEvent_t ev, uint32_t timeout_ms, bool *reached) {
  using clock = std::chrono::steady_clock;
  const auto deadline = clock::now() + std::chrono::milliseconds(timeout_ms);
  *reached = false;
  for (uint64_t spins = 0;; ++spins) {
    cudaError_t e = cudaEventQuery(ev);
    if (e == cudaSuccess) {
      *reached = true;
      return cudaSuccess;
    }
    if (e != cudaErrorNotReady) return e;
    if (timeout_ms == 0 || clock::now() >= deadline) return cudaSuccess;
    if (spins > 4000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_get_abi_version(uint32_t *abi_version, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  ullm_status_t st = validate_sink(error_sink);
  if (st != ULLM_STATUS_OK) return st;
  if (abi_version == nullptr)
    return write_error(error_sink, ULLM_STATUS_INVALID_ARGUMENT, "abi_version output is null");
  *abi_version = ULLM_CUDA_ABI_VERSION;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("ABI version query")
}

ullm_status_t ullm_cuda_query_version(ullm_cuda_version_info_t *version, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  ullm_status_t st = validate_sink(error_sink);
  if (st != ULLM_STATUS_OK) return st;
  st = validate_struct(version, error_sink, "version output");
  if (st != ULLM_STATUS_OK) return st;
  version->major = ULLM_CUDA_LIBRARY_VERSION_MAJOR;
  version->minor = ULLM_CUDA_LIBRARY_VERSION_MINOR;
  version->patch = ULLM_CUDA_LIBRARY_VERSION_PATCH;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("version query")
}

ullm_status_t ullm_cuda_backend_probe(uint32_t backend, ullm_cuda_backend_probe_result_t *result,
                                      ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  ullm_status_t st = validate_sink(error_sink);
  if (st != ULLM_STATUS_OK) return st;
  st = validate_struct(result, error_sink, "probe result");
  if (st != ULLM_STATUS_OK) return st;
  if (backend != ULLM_BACKEND_CUDA)
    return write_error(error_sink, ULLM_STATUS_UNSUPPORTED, "unknown backend identifier");
  result->backend = backend;
  result->available = 0U;
  result->cuda_runtime_present = 0U;
  result->device_count = 0U;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0) {
    (void)cudaGetLastError();
    return write_error(error_sink, ULLM_STATUS_CUDA_UNAVAILABLE,
                       "CUDA backend is unavailable: no usable device; no CPU fallback exists");
  }
  result->cuda_runtime_present = 1U;
  result->device_count = static_cast<uint32_t>(count);
  cudaDeviceProp prop;
  cudaError_t pe = cudaSuccess;
  const bool ok = device_is_target(0, &prop, &pe);
  if (pe == cudaSuccess) {
    result->sm_major = static_cast<uint32_t>(prop.major);
    result->sm_minor = static_cast<uint32_t>(prop.minor);
    result->sm_count = static_cast<uint32_t>(prop.multiProcessorCount);
    result->l2_bytes_mib = static_cast<uint32_t>(static_cast<size_t>(prop.l2CacheSize) >> 20);
    result->global_memory_bytes = static_cast<uint64_t>(prop.totalGlobalMem);
  }
  if (!ok)
    return write_error(error_sink, ULLM_STATUS_CUDA_UNAVAILABLE,
                       "CUDA backend is unavailable: device 0 is not compute capability 10.0 (the only "
                       "compiled target); no CPU fallback exists");
  result->available = 1U;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("backend probe")
}

ullm_status_t ullm_cuda_context_probe(const ullm_cuda_context_t *context,
                                      ullm_cuda_context_probe_result_t *result,
                                      ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  ullm_status_t st = validate_sink(error_sink);
  if (st != ULLM_STATUS_OK) return st;
  st = validate_struct(result, error_sink, "context probe result");
  if (st != ULLM_STATUS_OK) return st;
  result->context_present = context == nullptr ? 0U : 1U;
  result->cuda_available = 0U;
  result->device_ordinal = 0U;
  Context *c = as_context(context);
  if (c == nullptr)
    return write_error(error_sink, ULLM_STATUS_CUDA_UNAVAILABLE,
                       context == nullptr ? "no CUDA context was given" : "context handle is not live");
  result->cuda_available = 1U;
  result->device_ordinal = static_cast<uint32_t>(c->device);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("context probe")
}

ullm_status_t ullm_cuda_context_create(uint32_t device_ordinal, ullm_cuda_context_t **context,
                                       ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (context == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "context output is null");
  *context = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0) {
    (void)cudaGetLastError();
    return write_error(sink, ULLM_STATUS_CUDA_UNAVAILABLE,
                       "CUDA backend is unavailable: no usable device; no CPU fallback exists");
  }
  if (device_ordinal >= static_cast<uint32_t>(count))
    return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "device ordinal %u out of range (%d devices)", device_ordinal,
                  count);
  cudaDeviceProp prop;
  if (!device_is_target(static_cast<int>(device_ordinal), &prop, &e)) {
    if (e != cudaSuccess) return cuda_error(sink, e, "cudaGetDeviceProperties");
    return errorf(sink, ULLM_STATUS_CUDA_UNAVAILABLE,
                  "device %u is compute capability %d.%d; this library contains sm_100a code only and has no "
                  "CPU fallback",
                  device_ordinal, prop.major, prop.minor);
  }
  ULLM_CUDA_TRY(cudaSetDevice(static_cast<int>(device_ordinal)), "cudaSetDevice");
  Context *c = new (std::nothrow) Context();
  if (c == nullptr) return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  c->device = static_cast<int>(device_ordinal);
  c->sm_count = prop.multiProcessorCount;
  c->l2_bytes = static_cast<size_t>(prop.l2CacheSize);
  c->smem_optin = prop.sharedMemPerBlockOptin;
  // Mapped pinned memory: kernels write it only when a bounded wait expires, the host reads it
  // without a copy on every completion wait.
  e = cudaHostAlloc(reinterpret_cast<void **>(&c->host_flags), 16 * sizeof(uint32_t), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    std::memset(c->host_flags, 0, 16 * sizeof(uint32_t));
    e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&c->device_flags), c->host_flags, 0);
  }
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->abort_word), 256);
  if (e == cudaSuccess) e = cudaMemset(c->abort_word, 0, 256);
  if (e != cudaSuccess) {
    if (c->host_flags) (void)cudaFreeHost(c->host_flags);
    if (c->abort_word) (void)cudaFree(c->abort_word);
    (void)cudaGetLastError();
    delete c;
    return cuda_error(sink, e, "context flag allocation");
  }
  registry().add(c);
  *context = reinterpret_cast<ullm_cuda_context_t *>(c);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("context create")
}

ullm_status_t ullm_cuda_context_destroy(ullm_cuda_context_t **context, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (context == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "context pointer is null");
  Context *c = as_context(*context);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  if (c->live_children.load() != 0)
    return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "context still owns %llu queue/buffer/graph/comm/stack objects",
                  (unsigned long long)c->live_children.load());
  // Every queue, buffer, graph, comm and stack of the context is gone (those still retiring behind a
  // fence are counted as live), so no work of this context can be in flight: nothing to wait for.
  registry().remove(c);
  (void)cudaSetDevice(c->device);
  for (cudaEvent_t ev : c->event_pool) (void)cudaEventDestroy(ev);
  (void)cudaFreeHost(c->host_flags);
  (void)cudaFree(c->abort_word);
  c->magic = 0;
  delete c;
  *context = nullptr;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("context destroy")
}

ullm_status_t ullm_cuda_context_set_wait_limit(ullm_cuda_context_t *context, uint32_t limit_ms,
                                               ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Context *c = as_context(context);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  if (limit_ms == 0 || limit_ms > 600000U)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "the wait limit must be between 1 ms and 600000 ms");
  c->wait_limit_ms.store(limit_ms);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("context set wait limit")
}

ullm_status_t ullm_cuda_queue_create(ullm_cuda_context_t *context, ullm_cuda_queue_t **queue,
                                     ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (queue == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue output is null");
  *queue = nullptr;
  Context *c = as_context(context);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  ULLM_CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
  Queue *q = new (std::nothrow) Queue();
  if (q == nullptr) return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  q->ctx = c;
  cudaError_t e = cudaStreamCreateWithFlags(&q->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaHostAlloc(&q->staging, kStagingBytes, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    if (q->stream) (void)cudaStreamDestroy(q->stream);
    delete q;
    return cuda_error(sink, e, "queue create");
  }
  c->live_children++;
  {
    std::lock_guard<std::mutex> g(c->mutex);
    c->queues.push_back(q);
  }
  registry().add(q);
  *queue = reinterpret_cast<ullm_cuda_queue_t *>(q);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("queue create")
}

ullm_status_t ullm_cuda_queue_destroy(ullm_cuda_queue_t **queue, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (queue == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue pointer is null");
  Queue *q = as_queue(*queue);
  if (q == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "queue handle is not live");
  if (q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue is still capturing");
  registry().remove(q);
  Context *ctx = q->ctx;
  q->magic = 0;
  // The handle is dead from here on; the stream, its pinned staging and the GEMM scratch are released
  // as soon as the stream is observed idle (at once when it already is), never by blocking the caller.
  // Until then the stream stays on the context's list, so that a buffer freed meanwhile still waits for it.
  const bool watched = retire_behind(ctx->device, q->stream, [q, ctx] {
    {
      std::lock_guard<std::mutex> g(ctx->mutex);
      for (size_t i = 0; i < ctx->queues.size(); ++i)
        if (ctx->queues[i] == q) {
          ctx->queues.erase(ctx->queues.begin() + static_cast<long>(i));
          break;
        }
    }
    (void)cudaStreamDestroy(q->stream);
    (void)cudaFreeHost(q->staging);
    if (q->scratch.ptr != nullptr) (void)cudaFree(q->scratch.ptr);
    if (q->scratch.tile_counters != nullptr) (void)cudaFree(q->scratch.tile_counters);
    ctx->live_children--;
    delete q;
  });
  *queue = nullptr;
  if (!watched)
    return write_error(sink, ULLM_STATUS_CUDA_RUNTIME_ERROR,
                       "queue retired without proof of completion: its resources are abandoned, not freed");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("queue destroy")
}

ullm_status_t ullm_cuda_buffer_alloc(ullm_cuda_context_t *context, uint64_t size_bytes,
                                     ullm_cuda_buffer_t **buffer, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (buffer == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "buffer output is null");
  *buffer = nullptr;
  Context *c = as_context(context);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  if (size_bytes == 0) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "buffer size is zero");
  ULLM_CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
  Buffer *b = new (std::nothrow) Buffer();
  if (b == nullptr) return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  cudaError_t e = cudaMalloc(&b->ptr, static_cast<size_t>(size_bytes));
  if (e != cudaSuccess) {
    delete b;
    (void)cudaGetLastError();
    return cuda_error(sink, e, "cudaMalloc");
  }
  b->ctx = c;
  b->size = size_bytes;
  c->live_children++;
  registry().add(b);
  *buffer = reinterpret_cast<ullm_cuda_buffer_t *>(b);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("buffer alloc")
}

ullm_status_t ullm_cuda_buffer_free(ullm_cuda_buffer_t **buffer, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (buffer == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "buffer pointer is null");
  Buffer *b = as_buffer(*buffer);
  if (b == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "buffer handle is not live");
  registry().remove(b);
  Context *ctx = b->ctx;
  b->magic = 0;
  *buffer = nullptr;
  // Any queue of the context may still have work that uses the memory.  It is freed at once when every
  // queue is observed idle; otherwise the free waits, in the background, behind a fence on each busy queue.
  std::vector<cudaStream_t> busy;
  (void)cudaSetDevice(ctx->device);
  {
    std::lock_guard<std::mutex> g(ctx->mutex);
    for (Queue *q : ctx->queues)
      if (cudaStreamQuery(q->stream) != cudaSuccess) busy.push_back(q->stream);
  }
  (void)cudaGetLastError();
  auto remaining = std::make_shared<std::atomic<size_t>>(busy.size());
  auto release = [b, ctx] {
    (void)cudaFree(b->ptr);
    ctx->live_children--;
    delete b;
  };
  if (busy.empty()) {
    release();
    return ULLM_STATUS_OK;
  }
  bool watched = true;
  for (cudaStream_t s : busy)
    watched = retire_behind(ctx->device, s, [remaining, release] {
                if (remaining->fetch_sub(1) == 1) release();
              }) && watched;
  if (!watched)
    return write_error(sink, ULLM_STATUS_CUDA_RUNTIME_ERROR,
                       "buffer retired without proof of completion: its memory is abandoned, not freed");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("buffer free")
}

ullm_status_t ullm_cuda_buffer_size(const ullm_cuda_buffer_t *buffer, uint64_t *size_bytes,
                                    ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  ullm_status_t st = validate_sink(error_sink);
  if (st != ULLM_STATUS_OK) return st;
  Buffer *b = as_buffer(buffer);
  if (b == nullptr) return write_error(error_sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "buffer handle is not live");
  if (size_bytes == nullptr) return write_error(error_sink, ULLM_STATUS_INVALID_ARGUMENT, "size output is null");
  *size_bytes = b->size;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("buffer size")
}

static ullm_status_t copy_chunks(Queue *q, void *dev, void *host, uint64_t bytes, bool to_device, sink_t *sink) {
  if (q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "host copies cannot be captured");
  uint8_t *d = static_cast<uint8_t *>(dev);
  uint8_t *h = static_cast<uint8_t *>(host);
  uint64_t done = 0, copies = 0;
  while (done < bytes) {
    const size_t n = static_cast<size_t>(bytes - done < kStagingBytes ? bytes - done : kStagingBytes);
    if (to_device) {
      std::memcpy(q->staging, h + done, n);
      ULLM_CUDA_TRY(cudaMemcpyAsync(d + done, q->staging, n, cudaMemcpyHostToDevice, q->stream), "upload");
      ULLM_CUDA_TRY(cudaStreamSynchronize(q->stream), "upload synchronize");
    } else {
      ULLM_CUDA_TRY(cudaMemcpyAsync(q->staging, d + done, n, cudaMemcpyDeviceToHost, q->stream), "download");
      ULLM_CUDA_TRY(cudaStreamSynchronize(q->stream), "download synchronize");
      std::memcpy(h + done, q->staging, n);
    }
    done += n;
    ++copies;
  }
  std::lock_guard<std::mutex> g(q->mutex);
  q->copy_count += copies;
  return ULLM_STATUS_OK;
}

ullm_status_t ullm_cuda_buffer_upload(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t dst, const void *host_src,
                                      uint64_t size_bytes, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (size_bytes == 0) return ULLM_STATUS_OK;
  if (host_src == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "host source is null");
  void *d = nullptr;
  st = resolve(dst, size_bytes, 1, q->ctx, "upload destination", sink, &d);
  if (st != ULLM_STATUS_OK) return st;
  return copy_chunks(q, d, const_cast<void *>(host_src), size_bytes, true, sink);
  ULLM_ENTRY_END("buffer upload")
}

ullm_status_t ullm_cuda_buffer_download(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t src, void *host_dst,
                                        uint64_t size_bytes, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (size_bytes == 0) return ULLM_STATUS_OK;
  if (host_dst == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "host destination is null");
  void *d = nullptr;
  st = resolve(src, size_bytes, 1, q->ctx, "download source", sink, &d);
  if (st != ULLM_STATUS_OK) return st;
  return copy_chunks(q, d, host_dst, size_bytes, false, sink);
  ULLM_ENTRY_END("buffer download")
}

ullm_status_t ullm_cuda_buffer_fill(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t dst, uint8_t value,
                                    uint64_t size_bytes, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (size_bytes == 0) return ULLM_STATUS_OK;
  void *d = nullptr;
  st = resolve(dst, size_bytes, 1, q->ctx, "fill destination", sink, &d);
  if (st != ULLM_STATUS_OK) return st;
  ULLM_CUDA_TRY(cudaMemsetAsync(d, value, static_cast<size_t>(size_bytes), q->stream), "cudaMemsetAsync");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("buffer fill")
}

ullm_status_t ullm_cuda_queue_signal(ullm_cuda_queue_t *queue, ullm_cuda_completion_t **completion,
                                     ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (completion == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "completion output is null");
  *completion = nullptr;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "cannot signal while capturing");
  if (!submissions_open(sink, &st)) return st;
  cudaError_t e = cudaSuccess;
  cudaEvent_t ev = take_event(q->ctx, &e);
  if (e != cudaSuccess) return cuda_error(sink, e, "cudaEventCreate");
  e = cudaEventRecord(ev, q->stream);
  if (e != cudaSuccess) {
    give_event(q->ctx, ev);
    return cuda_error(sink, e, "cudaEventRecord");
  }
  Completion *c = new (std::nothrow) Completion();
  if (c == nullptr) {
    give_event(q->ctx, ev);
    return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  }
  c->queue = q;
  c->ctx = q->ctx;
  c->stream = q->stream;
  c->event = ev;
  {
    std::lock_guard<std::mutex> g(q->mutex);
    c->dispatch_count = q->dispatch_count;
    c->copy_count = q->copy_count;
    q->dispatch_count = 0;
    q->copy_count = 0;
  }
  q->ctx->live_children++;
  registry().add(c);
  *completion = reinterpret_cast<ullm_cuda_completion_t *>(c);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("queue signal")
}

static Completion *as_completion(const ullm_cuda_completion_t *h) {
  Completion *c = checked<Completion>(h);
  return (c && c->magic == kMagicCompletion) ? c : nullptr;
}

// The handle dies here.  Its event returns to the pool only when it has been observed reached; an event
// that may still be pending is destroyed instead (the runtime defers that until it completes), so that
// no later completion can be confused with this one.
static void retire_completion(Completion *c, bool reached) {
  registry().remove(c);
  if (reached)
    give_event(c->ctx, c->event);
  else
    (void)cudaEventDestroy(c->event);
  c->ctx->live_children--;
  c->magic = 0;
  delete c;
}

ullm_status_t ullm_cuda_completion_query(ullm_cuda_completion_t *completion, uint32_t timeout_ms,
                                         ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Completion *c = as_completion(completion);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "completion handle is not live");
  (void)cudaSetDevice(c->ctx->device);
  bool reached = false;
  cudaError_t e = poll_event(c->event, timeout_ms, &reached);
  if (e != cudaSuccess) return cuda_error(sink, e, "cudaEventQuery");
  if (!reached) return write_error(sink, ULLM_STATUS_CUDA_TIMEOUT, "completion not reached before the deadline");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("completion query")
}

ullm_status_t ullm_cuda_completion_wait(ullm_cuda_completion_t *completion, uint32_t timeout_ms,
                                        ullm_cuda_completion_result_t *result,
                                        ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (result != nullptr) {
    st = validate_struct(result, sink, "completion result");
    if (st != ULLM_STATUS_OK) return st;
  }
  Completion *c = as_completion(completion);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "completion handle is not live");
  Context *ctx = c->ctx;
  const Queue *c_queue = c->queue;
  (void)cudaSetDevice(ctx->device);
  bool reached = false;
  cudaError_t e = poll_event(c->event, timeout_ms, &reached);
  // Like the reference (hip_evidence_runtime.hip.cpp:691-716) the handle is consumed by EVERY outcome,
  // a timeout included: a caller cannot retry a wait.  Polling without consuming is ullm_cuda_completion_query.
  if (e != cudaSuccess) {
    retire_completion(c, false);
    return cuda_error(sink, e, "cudaEventQuery");
  }
  if (!reached) {
    retire_completion(c, false);
    return write_error(sink, ULLM_STATUS_CUDA_TIMEOUT, "completion not reached before the deadline; the handle is consumed");
  }
  cudaStream_t stream = as_queue(reinterpret_cast<const ullm_cuda_queue_t *>(c_queue)) != nullptr ? c->stream : nullptr;
  uint32_t flags[4] = {0, 0, 0, 0};
  const uint32_t any = take_device_flags(ctx, stream, flags);
  if (result != nullptr) {
    result->dispatch_count = c->dispatch_count;
    result->copy_count = c->copy_count;
    result->selected_backend = ULLM_BACKEND_CUDA;
    result->fallback_used = 0U;
    result->terminal = 1U;
    result->device_flags = any;
  }
  retire_completion(c, true);
  if (any != 0U)
    return errorf(sink, ULLM_STATUS_CUDA_DEVICE_FLAGGED,
                  "a kernel gave up a bounded wait (flags %08x %08x %08x %08x); results are not valid", flags[0],
                  flags[1], flags[2], flags[3]);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("completion wait")
}

ullm_status_t ullm_cuda_completion_elapsed_ms(ullm_cuda_completion_t *start, ullm_cuda_completion_t *end,
                                              float *milliseconds, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Completion *a = as_completion(start), *b = as_completion(end);
  if (a == nullptr || b == nullptr)
    return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "completion handle is not live");
  if (milliseconds == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "output is null");
  (void)cudaSetDevice(a->ctx->device);
  cudaError_t e = cudaEventElapsedTime(milliseconds, a->event, b->event);
  if (e == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return write_error(sink, ULLM_STATUS_CUDA_TIMEOUT, "completions not reached yet");
  }
  if (e != cudaSuccess) return cuda_error(sink, e, "cudaEventElapsedTime");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("completion elapsed")
}

ullm_status_t ullm_cuda_completion_destroy(ullm_cuda_completion_t **completion,
                                           ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (completion == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "completion pointer is null");
  if (*completion == nullptr) return ULLM_STATUS_OK;  // already consumed by wait and nulled by the caller
  Completion *c = as_completion(*completion);
  if (c == nullptr) {
    *completion = nullptr;  // consumed by a successful wait: destroying it again is harmless
    return ULLM_STATUS_OK;
  }
  (void)cudaSetDevice(c->ctx->device);
  retire_completion(c, cudaEventQuery(c->event) == cudaSuccess);
  (void)cudaGetLastError();
  *completion = nullptr;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("completion destroy")
}

ullm_status_t ullm_cuda_queue_capture_begin(ullm_cuda_queue_t *queue, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue is already capturing");
  ULLM_CUDA_TRY(cudaStreamBeginCapture(q->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
  q->capturing = true;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("capture begin")
}

ullm_status_t ullm_cuda_queue_capture_end(ullm_cuda_queue_t *queue, ullm_cuda_graph_t **graph,
                                          ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (graph == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "graph output is null");
  *graph = nullptr;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (!q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue is not capturing");
  q->capturing = false;
  cudaGraph_t g = nullptr;
  ULLM_CUDA_TRY(cudaStreamEndCapture(q->stream, &g), "cudaStreamEndCapture");
  Graph *gr = new (std::nothrow) Graph();
  if (gr == nullptr) {
    (void)cudaGraphDestroy(g);
    return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  }
  gr->ctx = q->ctx;
  gr->graph = g;
  size_t nodes = 0;
  (void)cudaGraphGetNodes(g, nullptr, &nodes);
  if (nodes != 0) {
    std::vector<cudaGraphNode_t> list(nodes);
    if (cudaGraphGetNodes(g, list.data(), &nodes) == cudaSuccess)
      for (size_t i = 0; i < nodes; ++i) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(list[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) gr->kernel_nodes++;
      }
  }
  cudaError_t e = cudaGraphInstantiate(&gr->exec, g, 0);
  if (e != cudaSuccess) {
    (void)cudaGraphDestroy(g);
    delete gr;
    return cuda_error(sink, e, "cudaGraphInstantiate");
  }
  // launches recorded during capture were counted as dispatches; they have not run
  {
    std::lock_guard<std::mutex> gq(q->mutex);
    q->dispatch_count = q->dispatch_count >= gr->kernel_nodes ? q->dispatch_count - gr->kernel_nodes : 0;
    q->total_dispatch = q->total_dispatch >= gr->kernel_nodes ? q->total_dispatch - gr->kernel_nodes : 0;
  }
  q->ctx->live_children++;
  registry().add(gr);
  *graph = reinterpret_cast<ullm_cuda_graph_t *>(gr);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("capture end")
}

ullm_status_t ullm_cuda_graph_launch(ullm_cuda_graph_t *graph, ullm_cuda_queue_t *queue,
                                     ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Graph *g = checked<Graph>(graph);
  if (g == nullptr || g->magic != kMagicGraph)
    return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "graph handle is not live");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (q->ctx != g->ctx) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "graph belongs to another context");
  ULLM_CUDA_TRY(cudaGraphLaunch(g->exec, q->stream), "cudaGraphLaunch");
  std::lock_guard<std::mutex> gq(q->mutex);
  q->dispatch_count += g->kernel_nodes;
  q->total_dispatch += g->kernel_nodes;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("graph launch")
}

ullm_status_t ullm_cuda_graph_destroy(ullm_cuda_graph_t **graph, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (graph == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "graph pointer is null");
  Graph *g = checked<Graph>(*graph);
  if (g == nullptr || g->magic != kMagicGraph)
    return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "graph handle is not live");
  registry().remove(g);
  (void)cudaSetDevice(g->ctx->device);
  // destroying an executable graph that is still running is legal: the runtime keeps what the launch needs
  (void)cudaGraphExecDestroy(g->exec);
  (void)cudaGraphDestroy(g->graph);
  g->ctx->live_children--;
  g->magic = 0;
  delete g;
  *graph = nullptr;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("graph destroy")
}

}  // extern "C"

// C++17 host mirror of the reference's safe wrapper crate (crates/ullm-hip/src/lib.rs) over the C ABI of
// ullm_cuda.h — what `ullm-cuda` would be in the Rust workspace, for hosts that are compiled code.
// Header-only; link against libullm_cuda.so.  Nothing here computes: every call goes through the C ABI.
//
//   reference (ullm-hip)                         here
//   Status::from_raw / raw      lib.rs:20-76     ullm::cuda::Status, status_from_raw
//   HipError{status,message}    lib.rs:78-110    ullm::cuda::Error (an exception; never crosses the C ABI)
//   512-byte stack sink         lib.rs:154-187   detail::Sink
//   abi_version/version/probes  lib.rs:189-273   abi_version(), version(), backend_probe()
//   EvidenceCompletion::wait    lib.rs:305-351   Completion::wait (consumed unless it times out)
//   HipBackend::connect         lib.rs:475-485   Backend::connect (needs an available probe)
//   impl Backend for HipBackend lib.rs:487-513   Backend::name / capabilities / supports
#pragma once

#include <chrono>
#include <cstdint>
#include <cstring>
#include <limits>
#include <optional>
#include <stdexcept>
#include <string>
#include <algorithm>
#include <utility>
#include <vector>

#include "ullm_cuda.h"

namespace ullm::cuda {

enum class Status : uint32_t {
  Ok = ULLM_STATUS_OK,
  InvalidArgument = ULLM_STATUS_INVALID_ARGUMENT,
  BufferTooSmall = ULLM_STATUS_BUFFER_TOO_SMALL,
  Unsupported = ULLM_STATUS_UNSUPPORTED,
  CudaUnavailable = ULLM_STATUS_CUDA_UNAVAILABLE,
  InvalidAbiVersion = ULLM_STATUS_INVALID_ABI_VERSION,
  ReservedNonzero = ULLM_STATUS_RESERVED_NONZERO,
  InternalError = ULLM_STATUS_INTERNAL_ERROR,
  Timeout = ULLM_STATUS_CUDA_TIMEOUT,
  InvalidHandle = ULLM_STATUS_CUDA_INVALID_HANDLE,
  ZeroDispatch = ULLM_STATUS_CUDA_ZERO_DISPATCH,
  RuntimeError = ULLM_STATUS_CUDA_RUNTIME_ERROR,
  DispatchContract = ULLM_STATUS_CUDA_DISPATCH_CONTRACT,
  OutOfMemory = ULLM_STATUS_CUDA_OUT_OF_MEMORY,
  OutOfRange = ULLM_STATUS_CUDA_OUT_OF_RANGE,
  CommError = ULLM_STATUS_CUDA_COMM_ERROR,
  DeviceFlagged = ULLM_STATUS_CUDA_DEVICE_FLAGGED,
  Unknown = 0xffffffffu,  // a code this header does not know (the raw value is kept in Error::raw)
};

inline Status status_from_raw(uint32_t raw) {
  switch (raw) {
    case ULLM_STATUS_OK:
    case ULLM_STATUS_INVALID_ARGUMENT:
    case ULLM_STATUS_BUFFER_TOO_SMALL:
    case ULLM_STATUS_UNSUPPORTED:
    case ULLM_STATUS_CUDA_UNAVAILABLE:
    case ULLM_STATUS_INVALID_ABI_VERSION:
    case ULLM_STATUS_RESERVED_NONZERO:
    case ULLM_STATUS_INTERNAL_ERROR:
    case ULLM_STATUS_CUDA_TIMEOUT:
    case ULLM_STATUS_CUDA_INVALID_HANDLE:
    case ULLM_STATUS_CUDA_ZERO_DISPATCH:
    case ULLM_STATUS_CUDA_RUNTIME_ERROR:
    case ULLM_STATUS_CUDA_DISPATCH_CONTRACT:
    case ULLM_STATUS_CUDA_OUT_OF_MEMORY:
    case ULLM_STATUS_CUDA_OUT_OF_RANGE:
    case ULLM_STATUS_CUDA_COMM_ERROR:
    case ULLM_STATUS_CUDA_DEVICE_FLAGGED:
      return static_cast<Status>(raw);
    default:
      return Status::Unknown;
  }
}

class Error : public std::runtime_error {
 public:
  Error(uint32_t raw, std::string message) : std::runtime_error(message), raw_(raw) {}
  Status status() const { return status_from_raw(raw_); }
  uint32_t raw() const { return raw_; }

 private:
  uint32_t raw_;
};

namespace detail {

// the caller-owned error sink: 512 bytes on the stack per call, as the reference wrapper does
struct Sink {
  char text[512];
  ullm_cuda_error_sink_t sink;
  Sink() {
    text[0] = '\0';
    std::memset(&sink, 0, sizeof(sink));
    sink.struct_size = sizeof(sink);
    sink.abi_version = ULLM_CUDA_ABI_VERSION;
    sink.message = text;
    sink.message_capacity = sizeof(text);
  }
  ullm_cuda_error_sink_t *get() { return &sink; }
  std::string message() const { return std::string(text); }
};

inline void check(uint32_t raw, const Sink &s) {
  if (raw != ULLM_STATUS_OK) throw Error(raw, s.message());
}

template <typename T>
T make_struct() {
  T v;
  std::memset(&v, 0, sizeof(v));
  v.struct_size = sizeof(T);
  v.abi_version = ULLM_CUDA_ABI_VERSION;
  return v;
}

}  // namespace detail

struct Version {
  uint32_t major, minor, patch;
};

struct BackendProbe {
  bool available;             // at least one sm_100 device is usable
  bool cuda_runtime_present;  // the CUDA runtime answered at all
  uint32_t device_count, sm_major, sm_minor, sm_count, l2_mib;
  uint64_t global_memory_bytes;
  std::string diagnostic;  // why not, when unavailable
};

inline uint32_t abi_version() {
  detail::Sink s;
  uint32_t v = 0;
  detail::check(ullm_cuda_get_abi_version(&v, s.get()), s);
  return v;
}

inline Version version() {
  detail::Sink s;
  auto info = detail::make_struct<ullm_cuda_version_info_t>();
  detail::check(ullm_cuda_query_version(&info, s.get()), s);
  return Version{info.major, info.minor, info.patch};
}

// CUDA_UNAVAILABLE from the probe is an answer, not a failure (lib.rs:230-242)
inline BackendProbe backend_probe() {
  detail::Sink s;
  auto r = detail::make_struct<ullm_cuda_backend_probe_result_t>();
  const uint32_t raw = ullm_cuda_backend_probe(ULLM_BACKEND_CUDA, &r, s.get());
  if (raw != ULLM_STATUS_OK && raw != ULLM_STATUS_CUDA_UNAVAILABLE) throw Error(raw, s.message());
  return BackendProbe{r.available != 0, r.cuda_runtime_present != 0, r.device_count, r.sm_major,    r.sm_minor,
                      r.sm_count,       r.l2_bytes_mib,              r.global_memory_bytes, s.message()};
}

// ---- owning handles (destroyed through the ABI; moves only) ---------------------------------------------

template <typename H, ullm_status_t (*Destroy)(H **, ullm_cuda_error_sink_t *)>
class Handle {
 public:
  Handle() = default;
  explicit Handle(H *h) : h_(h) {}
  Handle(Handle &&o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
  Handle &operator=(Handle &&o) noexcept {
    if (this != &o) {
      reset();
      h_ = std::exchange(o.h_, nullptr);
    }
    return *this;
  }
  Handle(const Handle &) = delete;
  Handle &operator=(const Handle &) = delete;
  ~Handle() { reset(); }
  H *get() const { return h_; }
  H *release() { return std::exchange(h_, nullptr); }
  void reset() {
    if (h_ != nullptr) {
      detail::Sink s;
      (void)Destroy(&h_, s.get());  // a destructor reports nothing
      h_ = nullptr;
    }
  }

 private:
  H *h_ = nullptr;
};

struct CompletionReport {
  uint64_t dispatch_count, copy_count;
  uint32_t selected_backend, fallback_used, device_flags;
};

class Completion {
 public:
  explicit Completion(ullm_cuda_completion_t *c) : h_(c) {}
  // Waits up to `timeout` and CONSUMES the completion whatever the outcome, like the reference's
  // Completion::wait(self, ..) (crates/ullm-hip/src/lib.rs:404-441): nullopt = not reached before the deadline
  // (the library has retired the handle; nothing can be retried on it).  The timeout saturates at u32::MAX
  // milliseconds and a sub-millisecond one is a single poll (lib.rs:400-402).  To poll without consuming use
  // reached().
  std::optional<CompletionReport> wait(std::chrono::nanoseconds timeout) {
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(timeout).count();
    const uint32_t t = ms <= 0 ? 0u : ms > (long long)std::numeric_limits<uint32_t>::max() ? std::numeric_limits<uint32_t>::max() : (uint32_t)ms;
    detail::Sink s;
    auto r = detail::make_struct<ullm_cuda_completion_result_t>();
    const uint32_t raw = ullm_cuda_completion_wait(h_.get(), t, &r, s.get());
    (void)h_.release();  // consumed by the library on every outcome
    if (raw == ULLM_STATUS_CUDA_TIMEOUT) return std::nullopt;
    detail::check(raw, s);
    return CompletionReport{r.dispatch_count, r.copy_count, r.selected_backend, r.fallback_used, r.device_flags};
  }
  // Single poll that keeps the completion.
  bool reached() {
    detail::Sink s;
    const uint32_t raw = ullm_cuda_completion_query(h_.get(), 0, s.get());
    if (raw == ULLM_STATUS_CUDA_TIMEOUT) return false;
    detail::check(raw, s);
    return true;
  }

 private:
  Handle<ullm_cuda_completion_t, ullm_cuda_completion_destroy> h_;
};

class Context {
 public:
  explicit Context(uint32_t device = 0) {
    detail::Sink s;
    ullm_cuda_context_t *c = nullptr;
    detail::check(ullm_cuda_context_create(device, &c, s.get()), s);
    h_ = Handle<ullm_cuda_context_t, ullm_cuda_context_destroy>(c);
  }
  ullm_cuda_context_t *get() const { return h_.get(); }

 private:
  Handle<ullm_cuda_context_t, ullm_cuda_context_destroy> h_;
};

class Buffer {
 public:
  Buffer(const Context &ctx, uint64_t bytes) {
    detail::Sink s;
    ullm_cuda_buffer_t *b = nullptr;
    detail::check(ullm_cuda_buffer_alloc(ctx.get(), bytes, &b, s.get()), s);
    h_ = Handle<ullm_cuda_buffer_t, ullm_cuda_buffer_free>(b);
  }
  ullm_cuda_tensor_t at(uint64_t offset_bytes = 0) const { return ullm_cuda_tensor_t{h_.get(), offset_bytes}; }

 private:
  Handle<ullm_cuda_buffer_t, ullm_cuda_buffer_free> h_;
};

// The quantised linear op as a value: the additive sibling of SemanticOp for this path (the existing Matmul
// rule rejects a bf16 x quantised-weight product, crates/ullm-core/src/op.rs:97-113).
struct QuantLinear {
  uint32_t encoding = ULLM_CUDA_ENCODING_FP8_CHANNEL;
  uint64_t m = 1, n = 0, k = 0;
  ullm_cuda_tensor_t weight_values{nullptr, 0}, weight_scales{nullptr, 0}, input{nullptr, 0}, output{nullptr, 0};
  uint32_t input_dtype = ULLM_CUDA_DTYPE_BF16, output_dtype = ULLM_CUDA_DTYPE_BF16;
  uint32_t prologue = 0, epilogue = ULLM_CUDA_EPILOGUE_NONE, kernel = ULLM_CUDA_KERNEL_AUTO;
  float rms_eps = 1e-5f;
  ullm_cuda_tensor_t norm_weight{nullptr, 0};  // RMSNorm prologue: bf16 gamma[K]
  ullm_cuda_tensor_t residual{nullptr, 0};     // f32 [M, N] added to the result

  ullm_cuda_linear_desc_t desc() const {
    auto d = detail::make_struct<ullm_cuda_linear_desc_t>();
    d.weight.encoding = encoding;
    d.weight.group_size = encoding == ULLM_CUDA_ENCODING_AQ4 ? ULLM_CUDA_AQ4_GROUP : encoding == ULLM_CUDA_ENCODING_NVFP4 ? ULLM_CUDA_NVFP4_BLOCK : 0;
    d.weight.n = n;
    d.weight.k = k;
    d.weight.values = weight_values;
    d.weight.scales = weight_scales;
    d.m = m;
    d.input = input;
    d.output = output;
    d.input_dtype = input_dtype;
    d.output_dtype = output_dtype;
    d.prologue = prologue;
    d.kernel = kernel;
    d.rms_eps = rms_eps;
    d.epilogue = epilogue;
    d.norm_weight = norm_weight;
    d.residual = residual;
    return d;
  }
};

class Queue {
 public:
  explicit Queue(const Context &ctx) {
    detail::Sink s;
    ullm_cuda_queue_t *q = nullptr;
    detail::check(ullm_cuda_queue_create(ctx.get(), &q, s.get()), s);
    h_ = Handle<ullm_cuda_queue_t, ullm_cuda_queue_destroy>(q);
  }
  void upload(ullm_cuda_tensor_t dst, const void *src, uint64_t bytes) {
    detail::Sink s;
    detail::check(ullm_cuda_buffer_upload(h_.get(), dst, src, bytes, s.get()), s);
  }
  void download(ullm_cuda_tensor_t src, void *dst, uint64_t bytes) {
    detail::Sink s;
    detail::check(ullm_cuda_buffer_download(h_.get(), src, dst, bytes, s.get()), s);
  }
  void quantize(ullm_cuda_tensor_t src_f32, const ullm_cuda_weight_t &w) {
    detail::Sink s;
    detail::check(ullm_cuda_quantize(h_.get(), src_f32, &w, s.get()), s);
  }
  // submit -> wait -> destroy: the completion token is the only way to observe the result
  Completion linear(const QuantLinear &op) {
    detail::Sink s;
    const ullm_cuda_linear_desc_t d = op.desc();
    ullm_cuda_completion_t *c = nullptr;
    detail::check(ullm_cuda_linear_submit(h_.get(), &d, &c, s.get()), s);
    return Completion(c);
  }
  ullm_cuda_queue_t *get() const { return h_.get(); }

 private:
  Handle<ullm_cuda_queue_t, ullm_cuda_queue_destroy> h_;
};

// ---- coarse command lists (docs/architecture/runtime.md:53-63, :77-79 of the reference) ---------------------
// prepare (metadata only, kernels chosen) -> submit (spans bound with access modes, behind other submissions'
// events) -> event (queried or waited on without being consumed).

enum class EventState : uint32_t { Pending = ULLM_CUDA_EVENT_PENDING, Success = ULLM_CUDA_EVENT_SUCCESS, Failure = ULLM_CUDA_EVENT_FAILURE };

class Event {
 public:
  explicit Event(ullm_cuda_event_t *e) : h_(e) {}
  EventState query() const {
    detail::Sink s;
    uint32_t state = ULLM_CUDA_EVENT_PENDING;
    detail::check(ullm_cuda_event_query(h_.get(), &state, s.get()), s);
    return static_cast<EventState>(state);
  }
  // false = not terminal before the deadline; the event stays usable either way
  bool wait(std::chrono::milliseconds timeout) const {
    detail::Sink s;
    const uint32_t raw = ullm_cuda_event_wait(h_.get(), (uint32_t)std::min<long long>(timeout.count(), 0xffffffffll), s.get());
    if (raw == ULLM_STATUS_CUDA_TIMEOUT) return false;
    detail::check(raw, s);
    return true;
  }
  ullm_cuda_event_t *get() const { return h_.get(); }

 private:
  Handle<ullm_cuda_event_t, ullm_cuda_event_destroy> h_;
};

struct Binding {
  uint32_t op_index, slot, access;
  ullm_cuda_tensor_t tensor;
};

class Prepared {
 public:
  // the ops' shapes, dtypes and fusions only: their spans are ignored here and bound at submit
  Prepared(const Context &ctx, const std::vector<QuantLinear> &ops) {
    std::vector<ullm_cuda_plan_op_t> raw;
    for (const QuantLinear &op : ops) {
      const ullm_cuda_linear_desc_t d = op.desc();
      auto o = detail::make_struct<ullm_cuda_plan_op_t>();
      o.encoding = d.weight.encoding;
      o.group_size = d.weight.group_size;
      o.n = d.weight.n;
      o.k = d.weight.k;
      o.m = d.m;
      o.input_dtype = d.input_dtype;
      o.output_dtype = d.output_dtype;
      o.prologue = d.prologue;
      o.epilogue = d.epilogue;
      o.kernel = d.kernel;
      o.rms_eps = d.rms_eps;
      o.flags = (op.norm_weight.buffer != nullptr ? ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT : 0u) |
                (op.residual.buffer != nullptr ? ULLM_CUDA_PLAN_OP_HAS_RESIDUAL : 0u);
      raw.push_back(o);
    }
    detail::Sink s;
    ullm_cuda_prepared_t *p = nullptr;
    detail::check(ullm_cuda_prepare(ctx.get(), raw.data(), (uint32_t)raw.size(), &p, s.get()), s);
    h_ = Handle<ullm_cuda_prepared_t, ullm_cuda_prepared_destroy>(p);
  }
  Event submit(const Queue &q, const std::vector<Binding> &bindings, const std::vector<const Event *> &wait_for = {}) const {
    std::vector<ullm_cuda_binding_t> raw;
    for (const Binding &b : bindings) {
      auto r = detail::make_struct<ullm_cuda_binding_t>();
      r.op_index = b.op_index;
      r.slot = b.slot;
      r.access = b.access;
      r.tensor = b.tensor;
      raw.push_back(r);
    }
    std::vector<ullm_cuda_event_t *> waits;
    for (const Event *e : wait_for) waits.push_back(e->get());
    detail::Sink s;
    ullm_cuda_event_t *ev = nullptr;
    detail::check(ullm_cuda_submit(q.get(), h_.get(), raw.data(), (uint32_t)raw.size(), waits.empty() ? nullptr : waits.data(),
                                   (uint32_t)waits.size(), &ev, s.get()),
                  s);
    return Event(ev);
  }

 private:
  Handle<ullm_cuda_prepared_t, ullm_cuda_prepared_destroy> h_;
};

// ---- the Backend surface of crates/ullm-core/src/backend.rs:5-24 -------------------------------------------

struct BackendCapabilities {
  bool metadata_only, numerical_execution;
  std::optional<uint64_t> max_materialization_bytes;
};

struct BackendSupport {
  bool supported;
  std::string reason;     // when not supported
  uint32_t kernel = 0;    // ULLM_CUDA_KERNEL_* the library would run
};

class Backend {
 public:
  // A typed backend handle is only constructible after an available probe (lib.rs:469-485).
  static Backend connect() {
    BackendProbe p = backend_probe();
    if (!p.available) throw Error(ULLM_STATUS_CUDA_UNAVAILABLE, p.diagnostic);
    return Backend();
  }
  static const char *name() { return "cuda"; }
  static BackendCapabilities capabilities() { return BackendCapabilities{false, true, std::nullopt}; }
  // Shape-only: no device is touched (Backend::supports, backend.rs:8).  Usable without connect().
  static BackendSupport supports(const QuantLinear &op) {
    detail::Sink s;
    const ullm_cuda_linear_desc_t d = op.desc();
    uint32_t kernel = 0;
    const uint32_t raw = ullm_cuda_linear_supports(&d, &kernel, s.get());
    if (raw == ULLM_STATUS_OK) return BackendSupport{true, std::string(), kernel};
    if (raw == ULLM_STATUS_UNSUPPORTED) return BackendSupport{false, s.message(), 0};
    throw Error(raw, s.message());
  }

 private:
  Backend() = default;
};

}  // namespace ullm::cuda

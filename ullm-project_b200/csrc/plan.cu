// Coarse command lists: prepare (copy metadata, choose kernels) / submit (bindings with access modes, dependency
// events) / event query and wait / context shutdown with drain.
//
// This is the call unit the reference's runtime design fixes for its C ABI — a prepared plan of several ops, not
// one call per kernel — and its ownership rules (docs/architecture/runtime.md:53-63, :77-79):
//   * prepare copies reusable metadata into library-owned storage at once and keeps no pointer into the caller's
//     arrays; kernels are chosen at prepare time, so a missing capability shows before anything runs;
//   * submit copies bindings, access modes (crates/ullm-core/src/handles.rs:12-16) and dependency events during
//     the call; a synchronous validation / enqueue failure is submit's own status;
//   * a failure after enqueue is stored in the completion event, which owns its diagnostic, and is read with
//     event_query / event_wait (pending, success and failure are distinguished);
//   * the context's executor owns every in-flight submission (the InFlightSubmission of handles.rs:100-145):
//     dropping the event does not end the watch; shutdown refuses new work, drains and collects terminal statuses.
#include "internal.hpp"

#include <chrono>
#include <new>
#include <thread>

namespace ullm {

constexpr uint32_t kMagicPrepared = 0x70726531U, kMagicEvent = 0x65767431U;
constexpr uint32_t kMaxPlanOps = 4096;

struct Prepared {
  uint32_t magic = kMagicPrepared;
  Context *ctx = nullptr;
  std::vector<ullm_cuda_plan_op_t> ops;   // copied at prepare time
  std::vector<uint32_t> kernels;          // chosen at prepare time
};

// One submission in flight.  Two owners: the caller's event handle and the context's executor; it is freed when
// both have let go (the executor lets go once it has observed the terminal state).
struct Submission {
  uint32_t magic = kMagicEvent;
  Context *ctx = nullptr;
  cudaEvent_t done = nullptr;
  cudaStream_t stream = nullptr;
  Queue *queue = nullptr;
  uint32_t state = ULLM_CUDA_EVENT_PENDING;
  ullm_status_t status = ULLM_STATUS_OK;  // terminal status, owned here together with its diagnostic
  std::string diagnostic;
  bool caller_holds = true, executor_holds = true;
};

namespace {

Prepared *as_prepared(const ullm_cuda_prepared_t *h) {
  Prepared *p = checked<Prepared>(h);
  return (p && p->magic == kMagicPrepared) ? p : nullptr;
}
Submission *as_event(const ullm_cuda_event_t *h) {
  Submission *s = checked<Submission>(h);
  return (s && s->magic == kMagicEvent) ? s : nullptr;
}

// Observes the submission once (ctx->mutex held by the caller): pending stays pending; a reached event becomes
// success, or failure when a kernel of the context recorded a wait that gave up.
void observe(Submission *s) {
  if (s->state != ULLM_CUDA_EVENT_PENDING) return;
  const cudaError_t e = cudaEventQuery(s->done);
  if (e == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return;
  }
  if (e != cudaSuccess) {
    s->state = ULLM_CUDA_EVENT_FAILURE;
    s->status = ULLM_STATUS_CUDA_RUNTIME_ERROR;
    s->diagnostic = std::string("cudaEventQuery: ") + cudaGetErrorName(e);
    (void)cudaGetLastError();
    return;
  }
  s->state = ULLM_CUDA_EVENT_SUCCESS;
}

void finish_observation(Submission *s) {  // outside ctx->mutex: take_device_flags locks it itself
  if (s->state != ULLM_CUDA_EVENT_SUCCESS || s->status != ULLM_STATUS_OK) return;
  uint32_t words[4] = {0, 0, 0, 0};
  const bool queue_live = as_queue(reinterpret_cast<const ullm_cuda_queue_t *>(s->queue)) != nullptr;
  if (take_device_flags(s->ctx, queue_live ? s->stream : nullptr, words) != 0U) {
    char text[160];
    std::snprintf(text, sizeof(text), "a kernel gave up a bounded wait (flags %08x %08x %08x %08x); results are not valid",
                  words[0], words[1], words[2], words[3]);
    s->state = ULLM_CUDA_EVENT_FAILURE;
    s->status = ULLM_STATUS_CUDA_DEVICE_FLAGGED;
    s->diagnostic = text;
  }
}

void release_if_unowned(Submission *s) {
  if (s->caller_holds || s->executor_holds) return;
  (void)cudaEventDestroy(s->done);
  s->ctx->live_children--;
  s->magic = 0;
  delete s;
}

// The executor's sweep: every submission that has reached a terminal state leaves the in-flight list.
void sweep(Context *ctx) {
  std::vector<Submission *> finished;
  {
    std::lock_guard<std::mutex> g(ctx->mutex);
    for (size_t i = 0; i < ctx->in_flight.size();) {
      Submission *s = ctx->in_flight[i];
      observe(s);
      if (s->state != ULLM_CUDA_EVENT_PENDING) {
        finished.push_back(s);
        ctx->in_flight.erase(ctx->in_flight.begin() + static_cast<long>(i));
      } else {
        ++i;
      }
    }
  }
  for (Submission *s : finished) {
    finish_observation(s);
    bool gone = false;
    {
      std::lock_guard<std::mutex> g(ctx->mutex);
      s->executor_holds = false;
      gone = !s->caller_holds;
    }
    if (gone) {
      registry().remove(s);
      release_if_unowned(s);
    }
  }
}

ullm_cuda_linear_desc_t desc_of(const ullm_cuda_plan_op_t &op) {
  ullm_cuda_linear_desc_t d{};
  d.struct_size = sizeof(d);
  d.abi_version = ULLM_CUDA_ABI_VERSION;
  d.weight.encoding = op.encoding;
  d.weight.group_size = op.group_size;
  d.weight.n = op.n;
  d.weight.k = op.k;
  d.m = op.m;
  d.input_dtype = op.input_dtype;
  d.output_dtype = op.output_dtype;
  d.prologue = op.prologue;
  d.epilogue = op.epilogue;
  d.kernel = op.kernel;
  d.rms_eps = op.rms_eps;
  return d;
}

bool same_span(const ullm_cuda_tensor_t &a, const ullm_cuda_tensor_t &b) {
  return a.buffer == b.buffer && a.offset_bytes == b.offset_bytes;
}

}  // namespace
}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_prepare(ullm_cuda_context_t *context, const ullm_cuda_plan_op_t *ops, uint32_t count,
                                ullm_cuda_prepared_t **prepared, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (prepared == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "prepared output is null");
  *prepared = nullptr;
  Context *ctx = as_context(context);
  if (ctx == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  if (ctx->closing.load()) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "the context is shutting down: no new plans");
  if (ops == nullptr || count == 0 || count > kMaxPlanOps)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "a plan holds between 1 and 4096 ops");
  Prepared *p = new (std::nothrow) Prepared();
  if (p == nullptr) return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  p->ctx = ctx;
  for (uint32_t i = 0; i < count; ++i) {
    st = validate_struct(&ops[i], sink, "plan op");
    if (st == ULLM_STATUS_OK && (ops[i].flags & ~(ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT | ULLM_CUDA_PLAN_OP_HAS_RESIDUAL)) != 0)
      st = write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "unknown plan op flag");
    uint32_t kernel = 0;
    if (st == ULLM_STATUS_OK) {
      ullm_cuda_linear_desc_t d = desc_of(ops[i]);
      // the flags stand for bindings that arrive with submit: a placeholder makes the shape rules see them
      if (ops[i].flags & ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT) d.norm_weight.buffer = reinterpret_cast<ullm_cuda_buffer_t *>(p);
      if (ops[i].flags & ULLM_CUDA_PLAN_OP_HAS_RESIDUAL) d.residual.buffer = reinterpret_cast<ullm_cuda_buffer_t *>(p);
      st = linear_shape_check(&d, &kernel, sink);
    }
    if (st != ULLM_STATUS_OK) {
      delete p;
      return st;  // the sink names the rule; the failing op is the first one that does not pass
    }
    p->ops.push_back(ops[i]);  // copied: the caller's array may go away
    p->kernels.push_back(kernel);
  }
  ctx->live_children++;
  registry().add(p);
  *prepared = reinterpret_cast<ullm_cuda_prepared_t *>(p);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("prepare")
}

ullm_status_t ullm_cuda_prepared_destroy(ullm_cuda_prepared_t **prepared, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (prepared == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "prepared pointer is null");
  Prepared *p = as_prepared(*prepared);
  if (p == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "prepared handle is not live");
  // a submission copies what it needs during submit, so nothing in flight refers to the plan
  registry().remove(p);
  p->ctx->live_children--;
  p->magic = 0;
  delete p;
  *prepared = nullptr;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("prepared destroy")
}

ullm_status_t ullm_cuda_submit(ullm_cuda_queue_t *queue, ullm_cuda_prepared_t *prepared,
                               const ullm_cuda_binding_t *bindings, uint32_t binding_count,
                               ullm_cuda_event_t *const *wait_events, uint32_t wait_count, ullm_cuda_event_t **event,
                               ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (event != nullptr) *event = nullptr;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  Prepared *p = as_prepared(prepared);
  if (p == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "prepared handle is not live");
  if (p->ctx != q->ctx) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "plan and queue belong to different contexts");
  Context *ctx = q->ctx;
  if (ctx->closing.load()) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "the context is shutting down: no new submissions");
  if (q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "a plan cannot be submitted into a stream capture");
  if (!submissions_open(sink, &st)) return st;
  if ((bindings == nullptr && binding_count != 0) || (wait_events == nullptr && wait_count != 0))
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "binding or event array is null");
  sweep(ctx);

  // ---- bindings: copied and checked during the call -------------------------------------------------------
  const size_t nops = p->ops.size();
  struct Bound {
    ullm_cuda_tensor_t t[6];
    uint32_t access[6];
    bool have[6];
  };
  std::vector<Bound> bound(nops);
  for (Bound &b : bound)
    for (int s = 0; s < 6; ++s) b.have[s] = false;
  for (uint32_t i = 0; i < binding_count; ++i) {
    const ullm_cuda_binding_t &b = bindings[i];
    st = validate_struct(&b, sink, "binding");
    if (st != ULLM_STATUS_OK) return st;
    if (b.reserved0 != 0) return write_error(sink, ULLM_STATUS_RESERVED_NONZERO, "binding: reserved fields must be zero");
    if (b.op_index >= nops) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "binding %u names op %u of a %zu-op plan", i, b.op_index, nops);
    if (b.slot > ULLM_CUDA_SLOT_RESIDUAL) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "binding %u: unknown slot", i);
    if (b.access < ULLM_CUDA_ACCESS_READ || b.access > ULLM_CUDA_ACCESS_READ_WRITE)
      return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "binding %u: unknown access mode", i);
    Bound &dst = bound[b.op_index];
    if (dst.have[b.slot]) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %u: slot %u is bound twice", b.op_index, b.slot);
    const ullm_cuda_plan_op_t &op = p->ops[b.op_index];
    if ((b.slot == ULLM_CUDA_SLOT_NORM_WEIGHT && !(op.flags & ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT)) ||
        (b.slot == ULLM_CUDA_SLOT_RESIDUAL && !(op.flags & ULLM_CUDA_PLAN_OP_HAS_RESIDUAL)))
      return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %u was prepared without slot %u", b.op_index, b.slot);
    dst.have[b.slot] = true;
    dst.t[b.slot] = b.tensor;
    dst.access[b.slot] = b.access;
  }
  std::vector<ullm_cuda_linear_desc_t> descs(nops);
  for (size_t i = 0; i < nops; ++i) {
    const ullm_cuda_plan_op_t &op = p->ops[i];
    const Bound &b = bound[i];
    const bool need[6] = {true, true, true, true, (op.flags & ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT) != 0,
                          (op.flags & ULLM_CUDA_PLAN_OP_HAS_RESIDUAL) != 0};
    for (int s = 0; s < 6; ++s)
      if (need[s] && !b.have[s]) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %zu: slot %d is not bound", i, s);
    // access modes: what the op does with each binding must be permitted by what the binding declares
    for (int s = 0; s < 6; ++s) {
      if (!b.have[s]) continue;
      const bool reads = s != (int)ULLM_CUDA_SLOT_OUTPUT, writes = s == (int)ULLM_CUDA_SLOT_OUTPUT;
      if (reads && !(b.access[s] & ULLM_CUDA_ACCESS_READ))
        return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %zu: slot %d is read but its binding does not permit reading", i, s);
      if (writes && !(b.access[s] & ULLM_CUDA_ACCESS_WRITE))
        return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %zu: the output binding does not permit writing", i);
    }
    const ullm_cuda_tensor_t &out = b.t[ULLM_CUDA_SLOT_OUTPUT];
    if (need[ULLM_CUDA_SLOT_RESIDUAL] && same_span(out, b.t[ULLM_CUDA_SLOT_RESIDUAL]) &&
        b.access[ULLM_CUDA_SLOT_OUTPUT] != ULLM_CUDA_ACCESS_READ_WRITE)
      return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %zu: an output that is also the residual must be bound READ_WRITE", i);
    for (int s : {(int)ULLM_CUDA_SLOT_WEIGHT_VALUES, (int)ULLM_CUDA_SLOT_WEIGHT_SCALES, (int)ULLM_CUDA_SLOT_INPUT,
                  (int)ULLM_CUDA_SLOT_NORM_WEIGHT})
      if (b.have[s] && same_span(out, b.t[s]))
        return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "op %zu: the output aliases slot %d, which the op reads while it writes", i, s);
    ullm_cuda_linear_desc_t d = desc_of(op);
    d.kernel = p->kernels[i];  // the kernel chosen at prepare time
    d.weight.values = b.t[ULLM_CUDA_SLOT_WEIGHT_VALUES];
    d.weight.scales = b.t[ULLM_CUDA_SLOT_WEIGHT_SCALES];
    d.input = b.t[ULLM_CUDA_SLOT_INPUT];
    d.output = out;
    if (need[ULLM_CUDA_SLOT_NORM_WEIGHT]) d.norm_weight = b.t[ULLM_CUDA_SLOT_NORM_WEIGHT];
    if (need[ULLM_CUDA_SLOT_RESIDUAL]) d.residual = b.t[ULLM_CUDA_SLOT_RESIDUAL];
    descs[i] = d;
  }
  // ---- dependency events (copied: only their native events are used, now) ---------------------------------
  std::vector<cudaEvent_t> deps;
  for (uint32_t i = 0; i < wait_count; ++i) {
    Submission *dep = as_event(wait_events[i]);
    if (dep == nullptr) return errorf(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "dependency event %u is not live", i);
    if (dep->ctx != ctx) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "dependency event %u belongs to another context", i);
    deps.push_back(dep->done);
  }
  Submission *sub = new (std::nothrow) Submission();
  if (sub == nullptr) return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  cudaError_t e = cudaEventCreateWithFlags(&sub->done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    delete sub;
    return cuda_error(sink, e, "cudaEventCreate");
  }
  for (cudaEvent_t d : deps) {
    e = cudaStreamWaitEvent(q->stream, d, 0);
    if (e != cudaSuccess) {
      (void)cudaEventDestroy(sub->done);
      delete sub;
      return cuda_error(sink, e, "cudaStreamWaitEvent");
    }
  }
  // ---- enqueue every op in order; the first failure is the submit's status (what was enqueued before it runs) ----
  for (size_t i = 0; i < nops; ++i) {
    st = enqueue_linear_desc(q, &descs[i], sink);
    if (st != ULLM_STATUS_OK) {
      (void)cudaEventDestroy(sub->done);
      delete sub;
      return st;
    }
  }
  e = cudaEventRecord(sub->done, q->stream);
  if (e != cudaSuccess) {
    (void)cudaEventDestroy(sub->done);
    delete sub;
    return cuda_error(sink, e, "cudaEventRecord");
  }
  sub->ctx = ctx;
  sub->queue = q;
  sub->stream = q->stream;
  sub->caller_holds = event != nullptr;
  ctx->live_children++;
  registry().add(sub);
  {
    std::lock_guard<std::mutex> g(ctx->mutex);
    ctx->in_flight.push_back(sub);
  }
  if (event != nullptr) *event = reinterpret_cast<ullm_cuda_event_t *>(sub);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("submit")
}

static ullm_status_t report(Submission *s, uint32_t *state, sink_t *sink) {
  if (state != nullptr) *state = s->state;
  if (s->state == ULLM_CUDA_EVENT_FAILURE) return write_error(sink, s->status, s->diagnostic.c_str());
  return ULLM_STATUS_OK;
}

ullm_status_t ullm_cuda_event_query(ullm_cuda_event_t *event, uint32_t *state, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (state == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "state output is null");
  Submission *s = as_event(event);
  if (s == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "event handle is not live");
  (void)cudaSetDevice(s->ctx->device);
  sweep(s->ctx);
  return report(s, state, sink);
  ULLM_ENTRY_END("event query")
}

ullm_status_t ullm_cuda_event_wait(ullm_cuda_event_t *event, uint32_t timeout_ms, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Submission *s = as_event(event);
  if (s == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "event handle is not live");
  (void)cudaSetDevice(s->ctx->device);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (uint64_t spins = 0;; ++spins) {  // polls with a deadline, never blocks without one
    sweep(s->ctx);
    if (s->state != ULLM_CUDA_EVENT_PENDING) return report(s, nullptr, sink);
    if (timeout_ms == 0 || std::chrono::steady_clock::now() >= deadline)
      return write_error(sink, ULLM_STATUS_CUDA_TIMEOUT, "the submission has not completed before the deadline");
    if (spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  ULLM_ENTRY_END("event wait")
}

ullm_status_t ullm_cuda_event_destroy(ullm_cuda_event_t **event, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (event == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "event pointer is null");
  Submission *s = as_event(*event);
  if (s == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "event handle is not live");
  (void)cudaSetDevice(s->ctx->device);
  bool gone = false;
  {
    std::lock_guard<std::mutex> g(s->ctx->mutex);
    s->caller_holds = false;
    gone = !s->executor_holds;
  }
  if (gone) {
    registry().remove(s);
    release_if_unowned(s);
  } else {
    // still in flight: the executor keeps watching it; only the caller's handle dies
    registry().remove(s);
  }
  *event = nullptr;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("event destroy")
}

ullm_status_t ullm_cuda_context_shutdown(ullm_cuda_context_t *context, uint32_t timeout_ms, uint32_t *failed_submissions,
                                         ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Context *ctx = as_context(context);
  if (ctx == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  (void)cudaSetDevice(ctx->device);
  ctx->closing.store(true);  // from here on prepare and submit are refused
  uint32_t failed = 0;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    // drain: take the terminal status of everything that has finished
    std::vector<Submission *> finished;
    size_t pending = 0;
    {
      std::lock_guard<std::mutex> g(ctx->mutex);
      for (size_t i = 0; i < ctx->in_flight.size();) {
        Submission *s = ctx->in_flight[i];
        observe(s);
        if (s->state != ULLM_CUDA_EVENT_PENDING) {
          finished.push_back(s);
          ctx->in_flight.erase(ctx->in_flight.begin() + static_cast<long>(i));
        } else {
          ++i;
        }
      }
      pending = ctx->in_flight.size();
    }
    for (Submission *s : finished) {
      finish_observation(s);
      if (s->state == ULLM_CUDA_EVENT_FAILURE) ++failed;
      bool gone = false;
      {
        std::lock_guard<std::mutex> g(ctx->mutex);
        s->executor_holds = false;
        gone = !s->caller_holds;
      }
      if (gone) release_if_unowned(s);  // (its handle left the registry when the caller dropped it)
    }
    if (pending == 0) break;
    if (std::chrono::steady_clock::now() >= deadline) {
      if (failed_submissions != nullptr) *failed_submissions = failed;
      return errorf(sink, ULLM_STATUS_CUDA_TIMEOUT, "%zu submissions are still in flight; call shutdown again", pending);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  if (failed_submissions != nullptr) *failed_submissions = failed;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("context shutdown")
}

}  // extern "C"

// The quantised linear op behind the C ABI: argument validation, kernel selection
// (CUDA-core matvec for one token, or up to four with AQ4; tcgen05 GEMM otherwise) and the submit -> wait shape.
//
// Reference anchors:
//   capability query before execution     crates/ullm-core/src/backend.rs:5-24 (Backend::supports)
//   kernel chosen by op / encoding / shape docs/architecture/runtime.md:83-91
//   submit returns a completion to wait on native/hip/src/evidence_abi.h:48-59
//   result report: backend id, dispatch count, fallback_used = 0   native/hip/src/evidence_abi.h:27-40
// The existing Matmul descriptor rule (same dtype and encoding on every operand,
// crates/ullm-core/src/op.rs:97-113) rejects a bf16 x quantised-weight product, so
// this op is an additive "quantised linear" kind with the weight stored [N,K].
#include "internal.hpp"

namespace ullm {

struct Resolved {
  LinearArgs args;
  uint32_t kernel = 0;
};

static ullm_status_t resolve_linear(const ullm_cuda_linear_desc_t *desc, const Context *ctx, bool need_buffers,
                                    sink_t *sink, Resolved *out) {
  ullm_status_t st = validate_struct(desc, sink, "linear descriptor");
  if (st != ULLM_STATUS_OK) return st;
  const ullm_cuda_weight_t &w = desc->weight;
  LinearArgs &a = out->args;
  if (desc->m == 0) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "M is zero");
  if (desc->m > (1u << 20)) return write_error(sink, ULLM_STATUS_UNSUPPORTED, "M above 2^20 is not supported");
  if (desc->input_dtype != ULLM_CUDA_DTYPE_BF16 && desc->input_dtype != ULLM_CUDA_DTYPE_F32)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "input dtype must be BF16 or F32");
  if (desc->output_dtype != ULLM_CUDA_DTYPE_BF16 && desc->output_dtype != ULLM_CUDA_DTYPE_F32)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "output dtype must be BF16 or F32");
  if (desc->prologue > ULLM_CUDA_PROLOGUE_SWIGLU)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "unknown prologue");
  if (desc->epilogue > ULLM_CUDA_EPILOGUE_SWIGLU)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "unknown epilogue");
  if (desc->epilogue == ULLM_CUDA_EPILOGUE_SWIGLU && (desc->weight.n % 2 != 0 || desc->output_dtype != ULLM_CUDA_DTYPE_BF16))
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "the SwiGLU epilogue needs an even N and a BF16 output");
  if (desc->kernel > ULLM_CUDA_KERNEL_GEMM) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "unknown kernel id");
  if (desc->prologue == ULLM_CUDA_PROLOGUE_RMSNORM && !(desc->rms_eps >= 0.0f))
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "rms_eps must be non-negative");
  if (desc->norm_weight.buffer != nullptr && desc->prologue != ULLM_CUDA_PROLOGUE_RMSNORM)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "norm_weight is only meaningful with the RMSNorm prologue");
  if (desc->residual.buffer != nullptr && desc->epilogue == ULLM_CUDA_EPILOGUE_SWIGLU)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "a residual cannot be combined with the SwiGLU epilogue");
  // Strides come from the caller: bound them so that no span computation below can wrap around.
  constexpr uint64_t kMaxStride = uint64_t(1) << 40;
  if (desc->input_row_stride > kMaxStride || desc->output_row_stride > kMaxStride || desc->residual_row_stride > kMaxStride)
    return write_error(sink, ULLM_STATUS_CUDA_OUT_OF_RANGE, "a row stride above 2^40 elements is not addressable");

  if (need_buffers) {
    WeightPtrs wp;
    st = resolve_weight(w, ctx, sink, &wp);
    if (st != ULLM_STATUS_OK) return st;
    a.w = wp.values;
    a.scales = wp.scales;
  } else {
    // shape-only validation: same rules as resolve_weight, without touching handles
    if (w.encoding != ULLM_CUDA_ENCODING_AQ4 && w.encoding != ULLM_CUDA_ENCODING_FP8_CHANNEL && w.encoding != ULLM_CUDA_ENCODING_NVFP4)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "weight encoding must be AQ4, FP8_CHANNEL or NVFP4");
    if (w.n == 0 || w.k == 0) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight has a zero extent");
    if (w.n > 0x7fffffffULL || w.k > 0x7fffffffULL)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "weight extents above 2^31-1 are not supported");
    if (w.encoding == ULLM_CUDA_ENCODING_AQ4 && (w.group_size != ULLM_CUDA_AQ4_GROUP || w.k % ULLM_CUDA_AQ4_GROUP))
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "AQ4 needs group size 128 and K a multiple of 128");
    if (w.encoding == ULLM_CUDA_ENCODING_NVFP4 && (w.group_size != ULLM_CUDA_NVFP4_BLOCK || w.k % 32))
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "NVFP4 needs block size 16 and K a multiple of 32");
    if (w.encoding == ULLM_CUDA_ENCODING_FP8_CHANNEL && (w.group_size != 0 || w.k % 16))
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "FP8_CHANNEL needs group_size 0 and K a multiple of 16");
  }
  a.m = static_cast<uint32_t>(desc->m);
  a.n = static_cast<uint32_t>(w.n);
  a.k = static_cast<uint32_t>(w.k);
  a.encoding = w.encoding;
  a.x_dtype = desc->input_dtype;
  a.y_dtype = desc->output_dtype;
  a.prologue = desc->prologue;
  a.rms_eps = desc->rms_eps;
  a.epilogue = desc->epilogue;
  const uint64_t out_cols = desc->epilogue == ULLM_CUDA_EPILOGUE_SWIGLU ? w.n / 2 : w.n;
  const uint64_t in_cols = desc->prologue == ULLM_CUDA_PROLOGUE_SWIGLU ? 2 * w.k : w.k;
  a.x_stride = desc->input_row_stride == 0 ? in_cols : desc->input_row_stride;
  a.y_stride = desc->output_row_stride == 0 ? out_cols : desc->output_row_stride;
  if (a.x_stride < in_cols) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "input row stride is shorter than a row");
  if (a.y_stride < out_cols) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "output row stride is shorter than a row");
  a.res_stride = desc->residual_row_stride == 0 ? out_cols : desc->residual_row_stride;
  if (a.res_stride < out_cols) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "residual row stride is shorter than a row");

  if (need_buffers) {
    const uint64_t xb = dtype_bytes(a.x_dtype), yb = dtype_bytes(a.y_dtype);
    // ((m - 1) * stride + cols) * bytes, checked: m <= 2^20, stride <= 2^40, cols < 2^32, bytes <= 4
    auto span = [&](uint64_t stride, uint64_t cols, uint64_t bytes, uint64_t *out_bytes) {
      uint64_t v = 0;
      return !__builtin_mul_overflow(desc->m - 1, stride, &v) && !__builtin_add_overflow(v, cols, &v) &&
             !__builtin_mul_overflow(v, bytes, out_bytes);
    };
    uint64_t x_bytes = 0, y_bytes = 0, r_bytes = 0;
    if (!span(a.x_stride, in_cols, xb, &x_bytes) || !span(a.y_stride, out_cols, yb, &y_bytes) ||
        !span(a.res_stride, out_cols, 4, &r_bytes))
      return write_error(sink, ULLM_STATUS_CUDA_OUT_OF_RANGE, "a tensor span does not fit 64 bits");
    void *x = nullptr, *y = nullptr;
    st = resolve(desc->input, x_bytes, xb, ctx, "linear input", sink, &x);
    if (st != ULLM_STATUS_OK) return st;
    st = resolve(desc->output, y_bytes, yb, ctx, "linear output", sink, &y);
    if (st != ULLM_STATUS_OK) return st;
    a.x = x;
    a.y = y;
    if (desc->norm_weight.buffer != nullptr) {
      void *g = nullptr;
      st = resolve(desc->norm_weight, w.k * 2, 16, ctx, "norm weight", sink, &g);
      if (st != ULLM_STATUS_OK) return st;
      a.norm_weight = g;
    }
    if (desc->residual.buffer != nullptr) {
      void *r = nullptr;
      st = resolve(desc->residual, r_bytes, 4, ctx, "residual", sink, &r);
      if (st != ULLM_STATUS_OK) return st;
      a.residual = static_cast<const float *>(r);
    }
    a.wait_limit_ms = ctx->wait_limit_ms.load();
    a.abort_word = ctx->abort_word;
  }

  const char *why_mv = "", *why_gemm = "";
  const bool nv = a.encoding == ULLM_CUDA_ENCODING_NVFP4;
  if (nv && (a.norm_weight != nullptr || desc->norm_weight.buffer != nullptr))
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "the NVFP4 decode kernel offers no prologue");
  const bool mv = nv ? nvfp4_matvec_supports(a, &why_mv) : matvec_supports(a, &why_mv);
  if (nv) why_gemm = "the tensor-core kernels do not take NVFP4 weights";
  const bool gm = !nv && gemm_supports(a, &why_gemm);
  uint32_t kernel = desc->kernel;
  if (kernel == ULLM_CUDA_KERNEL_AUTO)
    kernel = (mv && !(gm && auto_prefers_gemm(a))) ? ULLM_CUDA_KERNEL_MATVEC : (gm ? ULLM_CUDA_KERNEL_GEMM : 0u);
  if (kernel == ULLM_CUDA_KERNEL_MATVEC && !mv) return errorf(sink, ULLM_STATUS_UNSUPPORTED, "matvec: %s", why_mv);
  if (kernel == ULLM_CUDA_KERNEL_GEMM && !gm) return errorf(sink, ULLM_STATUS_UNSUPPORTED, "gemm: %s", why_gemm);
  if (kernel == 0u)
    return errorf(sink, ULLM_STATUS_UNSUPPORTED, "no kernel serves this shape (matvec: %s; gemm: %s); no CPU fallback",
                  why_mv, why_gemm);
  out->kernel = kernel;
  return ULLM_STATUS_OK;
}

// Validates a descriptor against the queue's context and enqueues it (the body of ullm_cuda_linear_enqueue; the
// command-list path submits every op of a plan through it).
ullm_status_t enqueue_linear_desc(Queue *q, const ullm_cuda_linear_desc_t *desc, sink_t *sink);
// Shape-only validation and kernel choice (the body of ullm_cuda_linear_supports; prepare uses it).
ullm_status_t linear_shape_check(const ullm_cuda_linear_desc_t *desc, uint32_t *kernel, sink_t *sink);

static ullm_status_t enqueue_resolved(Queue *q, const Resolved &r, sink_t *sink) {
  ullm_status_t refused = ULLM_STATUS_OK;
  if (!submissions_open(sink, &refused)) return refused;
  cudaError_t e = cudaSuccess;
  const int launched = r.kernel == ULLM_CUDA_KERNEL_MATVEC
                           ? (r.args.encoding == ULLM_CUDA_ENCODING_NVFP4 ? launch_matvec_nvfp4(q->ctx, q->stream, r.args, &e)
                                                                          : launch_matvec(q->ctx, q->stream, r.args, &e))
                           : launch_gemm(q->ctx, &q->scratch, q->stream, r.args, &e);
  if (launched < 0) return cuda_error(sink, e, "linear kernel launch");
  if (launched == 0)
    return write_error(sink, ULLM_STATUS_CUDA_ZERO_DISPATCH, "linear op launched no kernel");
  return end_launch(q, sink, "linear kernel launch", static_cast<uint64_t>(launched));
}

ullm_status_t enqueue_linear_desc(Queue *q, const ullm_cuda_linear_desc_t *desc, sink_t *sink) {
  Resolved r;
  ullm_status_t st = resolve_linear(desc, q->ctx, true, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  return enqueue_resolved(q, r, sink);
}

ullm_status_t linear_shape_check(const ullm_cuda_linear_desc_t *desc, uint32_t *kernel, sink_t *sink) {
  Resolved r;
  ullm_status_t st = resolve_linear(desc, nullptr, false, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  if (kernel != nullptr) *kernel = r.kernel;
  return ULLM_STATUS_OK;
}

}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_linear_supports(const ullm_cuda_linear_desc_t *desc, uint32_t *selected_kernel,
                                        ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Resolved r;
  st = resolve_linear(desc, nullptr, false, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  if (selected_kernel != nullptr) *selected_kernel = r.kernel;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("linear supports")
}

ullm_status_t ullm_cuda_linear_enqueue(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                       ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (desc == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "linear descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  Resolved r;
  st = resolve_linear(desc, q->ctx, true, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  return enqueue_resolved(q, r, sink);
  ULLM_ENTRY_END("linear enqueue")
}

ullm_status_t ullm_cuda_linear_enqueue_static_scratch(ullm_cuda_queue_t *queue,
                                                      const ullm_cuda_linear_desc_t *desc,
                                                      ullm_cuda_error_sink_t *error_sink) {
  // Allocation-free: the activation staging area is a fixed device array inside the library.
  // The first call on a device resolves that array's address (do it outside stream capture).
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (desc == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "linear descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  Resolved r;
  st = resolve_linear(desc, q->ctx, true, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  const char *why = "";
  if (!gemm_supports(r.args, &why)) return errorf(sink, ULLM_STATUS_UNSUPPORTED, "gemm: %s", why);
  if (!submissions_open(sink, &st)) return st;
  cudaError_t e = cudaSuccess;
  const int launched = launch_gemm_static_scratch(q->ctx, q->stream, r.args, &e);
  if (launched == -2)
    return errorf(sink, ULLM_STATUS_UNSUPPORTED,
                  "the allocation-free linear needs M*K*2 <= %llu bytes of staging (got %llu) and no SwiGLU epilogue",
                  (unsigned long long)ULLM_CUDA_STATIC_SCRATCH_BYTES,
                  (unsigned long long)r.args.m * r.args.k * 2ull);
  if (launched < 0) return cuda_error(sink, e, "allocation-free linear launch");
  return end_launch(q, sink, "allocation-free linear launch", static_cast<uint64_t>(launched));
  ULLM_ENTRY_END("linear enqueue (static scratch)")
}

// Common part of the two single-op halves of the fused all-reduce: the slots' span and the step word.
static ullm_status_t resolve_slots(const ullm_cuda_slots_t *sl, const Context *ctx, uint64_t pairs, sink_t *sink,
                                   uint8_t **base) {
  ullm_status_t st = validate_struct(sl, sink, "slots descriptor");
  if (st != ULLM_STATUS_OK) return st;
  if (sl->ranks == 0 || sl->ranks > static_cast<uint32_t>(kMaxPeers))
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "ranks must be between 1 and 8");
  if (sl->rank >= sl->ranks) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "rank must be below ranks");
  if (sl->gather > 1) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "gather must be 0 or 1");
  if (sl->rank_stride_bytes % 16 != 0 || sl->rank_stride_bytes < pairs * 8 || sl->rank_stride_bytes > (uint64_t(1) << 40))
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "rank_stride_bytes must be a multiple of 16 that holds M * cols pairs");
  void *p = nullptr;
  st = resolve(sl->slots, (sl->ranks - 1) * sl->rank_stride_bytes + pairs * 8, 16, ctx, "slots", sink, &p);
  if (st != ULLM_STATUS_OK) return st;
  *base = static_cast<uint8_t *>(p);
  return ULLM_STATUS_OK;
}

ullm_status_t ullm_cuda_linear_enqueue_partial(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                               const ullm_cuda_slots_t *slots, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (desc == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "linear descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  Resolved r;
  st = resolve_linear(desc, q->ctx, true, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  if (desc->epilogue != ULLM_CUDA_EPILOGUE_NONE || desc->residual.buffer != nullptr)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "a partial linear takes neither an epilogue nor a residual");
  const char *why = "";
  if (!matvec_supports(r.args, &why)) return errorf(sink, ULLM_STATUS_UNSUPPORTED, "matvec: %s", why);
  uint8_t *base = nullptr;
  st = resolve_slots(slots, q->ctx, static_cast<uint64_t>(r.args.m) * r.args.n, sink, &base);
  if (st != ULLM_STATUS_OK) return st;
  if (!submissions_open(sink, &st)) return st;
  LinearArgs a = r.args;
  // one device stands for every rank: each "peer" is the same buffer, the slot is chosen by rank * stride
  for (uint32_t p = 0; p < slots->ranks; ++p) a.push_out.peer_base[p] = base;
  a.push_out.slot_off[0] = a.push_out.slot_off[1] = 0;
  a.push_out.slot_stride = slots->rank_stride_bytes;
  a.push_out.step_counter = q->ctx->abort_word + 1;  // a word that stays zero: the tag is use + 1
  a.push_out.uses_per_step = 0;
  a.push_out.use = slots->tag - 1u;
  a.push_out.tp = 1;  // one store per value (all "peers" are this buffer)
  a.push_out.rank = slots->rank;
  cudaError_t e = cudaSuccess;
  const int launched = launch_matvec(q->ctx, q->stream, a, &e);
  if (launched < 0) return cuda_error(sink, e, "partial linear launch");
  return end_launch(q, sink, "partial linear launch", static_cast<uint64_t>(launched));
  ULLM_ENTRY_END("linear enqueue (partial)")
}

ullm_status_t ullm_cuda_linear_enqueue_reduced(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                               const ullm_cuda_slots_t *slots, ullm_cuda_tensor_t reduced_out,
                                               ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (desc == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "linear descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  // the residual of this entry belongs to the input ([M, K]): validate the rest of the descriptor without it
  ullm_cuda_linear_desc_t d = *desc;
  d.residual.buffer = nullptr;
  d.residual.offset_bytes = 0;
  d.residual_row_stride = 0;
  Resolved r;
  st = resolve_linear(&d, q->ctx, true, sink, &r);
  if (st != ULLM_STATUS_OK) return st;
  if (desc->prologue == ULLM_CUDA_PROLOGUE_SWIGLU)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "a reduced linear takes the NONE or RMSNORM prologue");
  if (r.args.k % 8 != 0) return write_error(sink, ULLM_STATUS_UNSUPPORTED, "a reduced linear needs K to be a multiple of 8");
  const char *why = "";
  if (!matvec_supports(r.args, &why)) return errorf(sink, ULLM_STATUS_UNSUPPORTED, "matvec: %s", why);
  uint8_t *base = nullptr;
  const uint64_t elems = static_cast<uint64_t>(r.args.m) * r.args.k;
  st = resolve_slots(slots, q->ctx, elems, sink, &base);
  if (st != ULLM_STATUS_OK) return st;
  LinearArgs a = r.args;
  if (desc->residual.buffer != nullptr) {
    if (desc->residual_row_stride != 0 && desc->residual_row_stride != r.args.k)
      return write_error(sink, ULLM_STATUS_UNSUPPORTED, "the input residual of a reduced linear is dense [M, K]");
    void *p = nullptr;
    st = resolve(desc->residual, elems * 4, 16, q->ctx, "input residual", sink, &p);
    if (st != ULLM_STATUS_OK) return st;
    a.push_in.residual = static_cast<const float *>(p);
  }
  if (reduced_out.buffer != nullptr) {
    void *p = nullptr;
    st = resolve(reduced_out, elems * 4, 16, q->ctx, "reduced output", sink, &p);
    if (st != ULLM_STATUS_OK) return st;
    a.push_in.reduced_out = static_cast<float *>(p);
  }
  if (!submissions_open(sink, &st)) return st;
  a.push_in.local_base = base;
  a.push_in.slot_off[0] = a.push_in.slot_off[1] = 0;
  a.push_in.slot_stride = slots->rank_stride_bytes;
  a.push_in.step_counter = q->ctx->abort_word + 1;
  a.push_in.uses_per_step = 0;
  a.push_in.use = slots->tag - 1u;
  a.push_in.tp = slots->ranks;
  a.push_in.cluster = slots->gather ? 8u : 0u;
  cudaError_t e = cudaSuccess;
  const int launched = launch_matvec(q->ctx, q->stream, a, &e);
  if (launched < 0) return cuda_error(sink, e, "reduced linear launch");
  return end_launch(q, sink, "reduced linear launch", static_cast<uint64_t>(launched));
  ULLM_ENTRY_END("linear enqueue (reduced)")
}

ullm_status_t ullm_cuda_linear_submit(ullm_cuda_queue_t *queue, const ullm_cuda_linear_desc_t *desc,
                                      ullm_cuda_completion_t **completion,
                                      ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (completion == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "completion output is null");
  *completion = nullptr;
  st = ullm_cuda_linear_enqueue(queue, desc, sink);
  if (st != ULLM_STATUS_OK) return st;
  return ullm_cuda_queue_signal(queue, completion, sink);
  ULLM_ENTRY_END("linear submit")
}

}  // extern "C"

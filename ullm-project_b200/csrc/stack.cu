// Linear stack of a decoder (per layer: fused QKV, O, gate+up, down; then the LM
// head), tensor-parallel across ranks, replayed as one CUDA graph per token count.
//
// New design: the reference has neither a model graph nor multi-GPU code
// (docs/plans/main-plan.md:55).  What it fixes is the shape of the boundary: work is
// enqueued on a queue and observed through a completion (docs/architecture/runtime.md:77-79).
//
// Dataflow of one step: the projections of a decoder block with their glue (no attention is computed;
// the first semantic ops the reference plans after its skeleton are exactly these:
// docs/plans/archive/2026/08/1-10/phase2-h3-g0-model-free-gpu.md:42):
//   h          = f32( input bf16 [m, hidden] )          the residual stream, fp32
//   qkv        = QKV( rmsnorm(bf16 h, g1) )             column-parallel, bf16 out
//   h          = h + O( qkv[:, :q_local] )              row-parallel, sum over ranks, residual add
//   act        = swiglu( GateUp( rmsnorm(bf16 h, g2) ) ) column-parallel rows [gate_l | up_l], bf16 out [m, ffn/tp]
//   h          = h + Down( act )                        row-parallel, sum over ranks, residual add
//   logits     = LMHead( rmsnorm(bf16 h, gf) )          column-parallel, bf16 out [m, vocab/tp]
// rmsnorm (with its weight vector) runs inside the consuming kernel's activation staging, swiglu in the
// producing kernel's epilogue, and the residual add either in the row-parallel kernel's epilogue (one GPU,
// or before an NCCL all-reduce on rank 0) or, with the fused all-reduce, in the consuming kernel's staging:
// "sum over ranks + residual + norm" is then one pass over the ranks' slots.
// h alternates between two fp32 buffers (a linear never updates its own residual in place: the blocks of a
// kernel read it while one of them writes the new value).
//
// Weights are generated on the device from (seed, tensor id, element index) and
// quantised there.  FP8 row-parallel shards are cut out of rows quantised over the
// FULL K, so that every tensor-parallel degree uses the same codes and scales.
#include "internal.hpp"

#include <cuda_bf16.h>

#include <chrono>
#include <cstdlib>
#include <map>
#include <new>
#include <thread>

namespace ullm {

namespace {

struct StackLinear {
  uint32_t which = 0, layer = 0;
  uint64_t tensor_id = 0;
  uint64_t full_n = 0, full_k = 0;
  uint64_t n = 0, k = 0;            // shard shape
  uint64_t row_begin = 0, col_begin = 0;
  uint64_t values_off = 0, scales_off = 0;  // into the weight buffer
  bool row_parallel = false;
  uint32_t prologue = 0, epilogue = 0, x_dtype = 0, y_dtype = 0;
  uint64_t in_off = 0, out_off = 0;  // into the activation buffer
  uint64_t x_stride = 0, y_stride = 0;
  bool out_is_step_output = false;
  bool has_norm = false, has_residual = false;
  uint64_t norm_off = 0;       // bf16 gamma[K] in the weight buffer
  uint64_t norm_tensor_id = 0;
  uint64_t res_off = 0;        // fp32 residual [m, hidden] in the activation buffer (row-parallel linears)
};

}  // namespace

struct Stack {
  uint32_t magic = kMagicStack;
  Context *ctx = nullptr;
  Queue *queue = nullptr;
  cudaStream_t stream = nullptr;  // the queue's, kept so that destruction does not touch a queue handle that died first
  Comm *comm = nullptr;
  ullm_cuda_stack_desc_t desc{};
  std::vector<StackLinear> linears;
  Buffer *weights = nullptr;   // registered buffers so that linear_info can hand out spans
  Buffer *acts = nullptr;
  Buffer *io = nullptr;        // [input | output]
  uint64_t io_out_off = 0;
  uint64_t weight_bytes = 0;
  void *pinned_in = nullptr, *pinned_out = nullptr;
  cudaEvent_t done = nullptr;
  std::map<uint32_t, cudaGraphExec_t> graphs;
  std::map<uint32_t, cudaGraph_t> graph_defs;
  uint64_t launches_per_step = 0;
  // fused all-reduce over peer memory (decode path): a ring of sites inside the symmetric buffer
  bool push = false;
  static constexpr uint32_t kRing = 4;
  uint64_t ring_slot_off[kRing][2] = {};
  uint64_t step_counter_off = 0;        // local word bumped once per step
  uint64_t slot_stride = 0;
  uint32_t sites = 0;                   // row-parallel linears per step
  uint32_t gather_cluster = 0;          // non-zero: consumers gather the ranks' slots once per cluster
  uint64_t h0_off = 0;                  // fp32 copy of the step input (the residual stream's first value)
};

namespace {

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// First kernel of every step: the bf16 input becomes the fp32 residual stream, and (fused all-reduce) the step
// counter every tag of the step derives from is bumped.
__global__ void step_begin_kernel(const __nv_bfloat16 *in, float *h, uint64_t count, uint32_t *counter) {
  if (counter != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *counter += 1u;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    h[i] = __bfloat162float(in[i]);
}

// gamma[i] = bf16(1 + z(seed, tensor, i) / 8), z the same counter-based normal stream the weights use
__global__ void gamma_kernel(const float *z, __nv_bfloat16 *out, uint64_t count) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(1.0f + z[i] * 0.125f);
}

uint64_t values_bytes(uint32_t enc, uint64_t n, uint64_t k) { return enc == ULLM_CUDA_ENCODING_AQ4 ? n * (k / 2) : n * k; }
uint64_t scales_bytes(uint32_t enc, uint64_t n, uint64_t k) {
  return enc == ULLM_CUDA_ENCODING_AQ4 ? n * (k / 128) * 2 : n * 4;
}

Buffer *make_buffer(Context *ctx, uint64_t bytes, cudaError_t *err) {
  Buffer *b = new (std::nothrow) Buffer();
  if (b == nullptr) {
    *err = cudaErrorMemoryAllocation;
    return nullptr;
  }
  *err = cudaMalloc(&b->ptr, static_cast<size_t>(bytes));
  if (*err != cudaSuccess) {
    delete b;
    return nullptr;
  }
  b->ctx = ctx;
  b->size = bytes;
  ctx->live_children++;
  registry().add(b);
  return b;
}

// Copies columns [c0, c0+cols) of a row-major [rows, full_cols] byte matrix.
cudaError_t copy_columns(cudaStream_t s, uint8_t *dst, const uint8_t *src, uint64_t rows, uint64_t full_cols,
                         uint64_t c0, uint64_t cols) {
  return cudaMemcpy2DAsync(dst, cols, src + c0, full_cols, cols, rows, cudaMemcpyDeviceToDevice, s);
}

// Generates and quantises one shard.  Row pieces of the full weight are listed in
// `pieces` as (first full row, row count); their shard rows are consecutive.
cudaError_t build_weight(Stack *st, const StackLinear &L, const std::vector<std::pair<uint64_t, uint64_t>> &pieces,
                         float *scratch_f32, uint8_t *scratch_codes, uint64_t scratch_elems) {
  cudaStream_t s = st->queue->stream;
  const uint32_t enc = st->desc.encoding;
  uint8_t *wbase = static_cast<uint8_t *>(st->weights->ptr);
  uint8_t *values = wbase + L.values_off;
  uint8_t *scales = wbase + L.scales_off;
  const bool full_rows = L.row_parallel && enc == ULLM_CUDA_ENCODING_FP8_CHANNEL && L.k != L.full_k;
  const uint64_t gen_k = full_rows ? L.full_k : L.k;
  const uint64_t gen_c0 = full_rows ? 0 : L.col_begin;
  uint64_t shard_row = 0;
  for (const auto &pc : pieces) {
    uint64_t done = 0;
    while (done < pc.second) {
      uint64_t rows = scratch_elems / gen_k;
      if (rows == 0) return cudaErrorInvalidValue;
      if (rows > pc.second - done) rows = pc.second - done;
      launch_synth_weight_tile(s, st->desc.seed, L.tensor_id, L.full_k, pc.first + done, gen_c0, rows, gen_k, 0.02f,
                               scratch_f32);
      uint8_t *v_dst = values + (enc == ULLM_CUDA_ENCODING_AQ4 ? shard_row * (L.k / 2) : shard_row * L.k);
      uint8_t *s_dst = scales + (enc == ULLM_CUDA_ENCODING_AQ4 ? shard_row * (L.k / 128) * 2 : shard_row * 4);
      if (full_rows) {
        launch_quantize(s, scratch_f32, enc, rows, gen_k, scratch_codes, s_dst);
        cudaError_t e = copy_columns(s, v_dst, scratch_codes, rows, L.full_k, L.col_begin, L.k);
        if (e != cudaSuccess) return e;
      } else {
        launch_quantize(s, scratch_f32, enc, rows, gen_k, v_dst, s_dst);
      }
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      done += rows;
      shard_row += rows;
    }
  }
  return cudaStreamSynchronize(s);
}

LinearArgs make_args(const Stack *st, const StackLinear &L, uint32_t m) {
  LinearArgs a;
  const uint8_t *wbase = static_cast<const uint8_t *>(st->weights->ptr);
  uint8_t *abase = static_cast<uint8_t *>(st->acts->ptr);
  uint8_t *iobase = static_cast<uint8_t *>(st->io->ptr);
  a.w = wbase + L.values_off;
  a.scales = wbase + L.scales_off;
  a.x = abase + L.in_off;
  a.y = L.out_is_step_output ? iobase + st->io_out_off : abase + L.out_off;
  a.m = m;
  a.n = static_cast<uint32_t>(L.n);
  a.k = static_cast<uint32_t>(L.k);
  a.x_stride = L.x_stride;
  a.y_stride = L.y_stride;
  a.encoding = st->desc.encoding;
  a.x_dtype = L.x_dtype;
  a.y_dtype = L.y_dtype;
  a.prologue = L.prologue;
  a.epilogue = L.epilogue;
  a.rms_eps = st->desc.rms_eps;
  a.norm_weight = L.has_norm ? wbase + L.norm_off : nullptr;
  a.residual = L.has_residual ? reinterpret_cast<const float *>(abase + L.res_off) : nullptr;
  a.res_stride = L.y_stride;
  a.wait_limit_ms = st->ctx->wait_limit_ms.load();
  a.abort_word = st->ctx->abort_word;
  return a;
}

// The fused all-reduce lives in the matvec kernels: a step uses it only when every linear of the step is served
// by them at this token count (otherwise the whole step sums with NCCL, the same verdict on every rank, which
// all build the same shapes).
bool step_can_push(const Stack *st, uint32_t m) {
  if (!st->push || m > 8) return false;
  for (const StackLinear &L : st->linears) {
    const char *why = "";
    if (!matvec_supports(make_args(st, L, m), &why)) return false;
  }
  return true;
}

// Enqueues every kernel of one step on the stack's stream; returns launches or -1.
int64_t enqueue_step(Stack *st, uint32_t m, cudaError_t *err, std::string *why) {
  cudaStream_t s = st->queue->stream;
  int64_t launches = 0;
  const uint32_t tp = st->desc.tp_size;
  const bool push = step_can_push(st, m);
  {
    uint8_t *abase = static_cast<uint8_t *>(st->acts->ptr);
    const uint64_t count = (uint64_t)m * st->desc.hidden;
    uint32_t *counter = push ? reinterpret_cast<uint32_t *>(comm_sym_ptr(st->comm, st->desc.tp_rank) + st->step_counter_off) : nullptr;
    const unsigned blocks = (unsigned)((count + 1023) / 1024 > 64 ? 64 : (count + 1023) / 1024);
    step_begin_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(st->io->ptr),
                                             reinterpret_cast<float *>(abase + st->h0_off), count, counter);
    *err = cudaGetLastError();
    if (*err != cudaSuccess) {
      if (why) *why = "step begin launch failed";
      return -1;
    }
    ++launches;
  }
  uint32_t site = 0;                      // row-parallel linears seen so far in this step
  bool consume = false;                   // the previous linear pushed: this one sums the slots
  const float *pending_residual = nullptr;  // ... and adds the residual the pushing linear left to it
  float *pending_out = nullptr;
  for (const StackLinear &L : st->linears) {
    LinearArgs a = make_args(st, L, m);
    // with several ranks the residual enters the sum exactly once: on rank 0 before an NCCL all-reduce, in the
    // consumer's staging with the fused all-reduce
    if (L.row_parallel && tp > 1 && (push || st->desc.tp_rank != 0)) a.residual = nullptr;
    if (push && (consume || L.row_parallel)) {
      uint8_t *local = comm_sym_ptr(st->comm, st->desc.tp_rank);
      const uint32_t *counter = reinterpret_cast<const uint32_t *>(local + st->step_counter_off);
      auto uses_of = [&](uint32_t r) { return (st->sites - r + Stack::kRing - 1) / Stack::kRing; };
      if (consume) {
        const uint32_t r = (site - 1) % Stack::kRing;
        a.push_in.local_base = local;
        a.push_in.slot_off[0] = st->ring_slot_off[r][0];
        a.push_in.slot_off[1] = st->ring_slot_off[r][1];
        a.push_in.slot_stride = st->slot_stride;
        a.push_in.step_counter = counter;
        a.push_in.uses_per_step = uses_of(r);
        a.push_in.use = (site - 1) / Stack::kRing;
        a.push_in.residual = pending_residual;
        a.push_in.reduced_out = pending_out;  // keeps residual + sum: the next residual, and readable by tests
        a.push_in.tp = tp;
        a.push_in.cluster = st->gather_cluster;
      }
      if (L.row_parallel) {
        const uint32_t r = site % Stack::kRing;
        for (uint32_t q = 0; q < tp; ++q) a.push_out.peer_base[q] = comm_sym_ptr(st->comm, q);
        a.push_out.slot_off[0] = st->ring_slot_off[r][0];
        a.push_out.slot_off[1] = st->ring_slot_off[r][1];
        a.push_out.slot_stride = st->slot_stride;
        a.push_out.step_counter = counter;
        a.push_out.uses_per_step = uses_of(r);
        a.push_out.use = site / Stack::kRing;
        a.push_out.tp = tp;
        a.push_out.rank = st->desc.tp_rank;
        uint8_t *abase = static_cast<uint8_t *>(st->acts->ptr);
        pending_residual = L.has_residual ? reinterpret_cast<const float *>(abase + L.res_off) : nullptr;
        pending_out = reinterpret_cast<float *>(abase + L.out_off);
      }
    }
    consume = push && L.row_parallel;
    if (L.row_parallel) ++site;
    const char *reason = "";
    int n;
    // the fused all-reduce lives in the matvec kernels; without it the faster kernel for the token count runs
    const char *reason_gemm = "";
    const bool mv = matvec_supports(a, &reason);
    if (mv && (push || !(gemm_supports(a, &reason_gemm) && auto_prefers_gemm(a)))) {
      n = launch_matvec(st->ctx, s, a, err);
    } else if (gemm_supports(a, &reason)) {
      n = launch_gemm(st->ctx, &st->queue->scratch, s, a, err);
    } else {
      *err = cudaErrorNotSupported;
      if (why) *why = std::string("no kernel serves a stack linear: ") + reason;
      return -1;
    }
    if (n < 0) {
      if (why) *why = "linear kernel launch failed";
      return -1;
    }
    launches += n;
    if (L.row_parallel && tp > 1 && !push) {
      std::string nccl_why;
      *err = comm_all_reduce_raw(st->comm, s, a.y, static_cast<uint64_t>(m) * L.y_stride, ULLM_CUDA_DTYPE_F32, &nccl_why);
      if (*err != cudaSuccess) {
        if (why) *why = "all-reduce failed: " + nccl_why;
        return -1;
      }
      launches += 1;
    }
  }
  *err = cudaSuccess;
  return launches;
}

ullm_status_t run_step(Stack *st, uint32_t m, sink_t *sink) {
  ullm_status_t refused = ULLM_STATUS_OK;
  if (!submissions_open(sink, &refused)) return refused;
  if (as_queue(reinterpret_cast<const ullm_cuda_queue_t *>(st->queue)) == nullptr)
    return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "the stack's queue has been destroyed");
  cudaStream_t s = st->queue->stream;
  cudaError_t e = cudaSuccess;
  std::string why;
  if (st->desc.flags & ULLM_CUDA_STACK_FLAG_NO_GRAPH) {
    const int64_t n = enqueue_step(st, m, &e, &why);
    if (n < 0) return errorf(sink, e == cudaErrorNotSupported ? ULLM_STATUS_UNSUPPORTED : ULLM_STATUS_CUDA_RUNTIME_ERROR,
                             "%s (%s)", why.c_str(), cudaGetErrorName(e));
    st->launches_per_step = static_cast<uint64_t>(n);
  } else {
    auto it = st->graphs.find(m);
    if (it == st->graphs.end()) {
      ULLM_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
      const int64_t n = enqueue_step(st, m, &e, &why);
      cudaGraph_t g = nullptr;
      cudaError_t ce = cudaStreamEndCapture(s, &g);
      if (n < 0) {
        if (g) (void)cudaGraphDestroy(g);
        (void)cudaGetLastError();
        return errorf(sink, e == cudaErrorNotSupported ? ULLM_STATUS_UNSUPPORTED : ULLM_STATUS_CUDA_RUNTIME_ERROR,
                      "%s (%s)", why.c_str(), cudaGetErrorName(e));
      }
      if (ce != cudaSuccess) return cuda_error(sink, ce, "cudaStreamEndCapture");
      cudaGraphExec_t ex = nullptr;
      ce = cudaGraphInstantiate(&ex, g, 0);
      if (ce != cudaSuccess) {
        (void)cudaGraphDestroy(g);
        return cuda_error(sink, ce, "cudaGraphInstantiate");
      }
      st->graphs[m] = ex;
      st->graph_defs[m] = g;
      st->launches_per_step = static_cast<uint64_t>(n);
      it = st->graphs.find(m);
    }
    ULLM_CUDA_TRY(cudaGraphLaunch(it->second, s), "cudaGraphLaunch");
  }
  std::lock_guard<std::mutex> g(st->queue->mutex);
  st->queue->dispatch_count += st->launches_per_step;
  st->queue->total_dispatch += st->launches_per_step;
  return ULLM_STATUS_OK;
}

Stack *as_stack(const ullm_cuda_stack_t *h) {
  Stack *s = checked<Stack>(h);
  return (s && s->magic == kMagicStack) ? s : nullptr;
}

// Never blocks: graphs may be destroyed while they run, everything a running step may still touch (weights,
// activations, pinned staging) is released once the queue's last work is observed complete.  `counted` = the
// stack was registered as a child of its context.
bool destroy_stack(Stack *st, bool counted) {
  (void)cudaSetDevice(st->ctx->device);
  for (auto &kv : st->graphs) (void)cudaGraphExecDestroy(kv.second);
  for (auto &kv : st->graph_defs) (void)cudaGraphDestroy(kv.second);
  st->graphs.clear();
  st->graph_defs.clear();
  st->magic = 0;
  if (st->comm != nullptr && st->push && as_comm(reinterpret_cast<const ullm_cuda_comm_t *>(st->comm)) != nullptr)
    comm_sym_release(st->comm);
  for (Buffer *b : {st->weights, st->acts, st->io})
    if (b != nullptr) registry().remove(b);  // the spans handed out by linear_info die with the stack
  Context *ctx = st->ctx;
  return retire_behind(ctx->device, st->stream, [st, ctx, counted] {
    if (st->done) (void)cudaEventDestroy(st->done);
    if (st->pinned_in) (void)cudaFreeHost(st->pinned_in);
    if (st->pinned_out) (void)cudaFreeHost(st->pinned_out);
    for (Buffer *b : {st->weights, st->acts, st->io})
      if (b != nullptr) {
        (void)cudaFree(b->ptr);
        ctx->live_children--;
        b->magic = 0;
        delete b;
      }
    if (counted) ctx->live_children--;
    delete st;
  });
}

}  // namespace
}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_stack_create(ullm_cuda_context_t *context, ullm_cuda_queue_t *queue,
                                     ullm_cuda_comm_t *comm, const ullm_cuda_stack_desc_t *desc,
                                     ullm_cuda_stack_t **stack, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (stack == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "stack output is null");
  *stack = nullptr;
  st = validate_struct(desc, sink, "stack descriptor");
  if (st != ULLM_STATUS_OK) return st;
  Context *ctx = as_context(context);
  if (ctx == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (q->ctx != ctx) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue belongs to another context");
  const ullm_cuda_stack_desc_t &d = *desc;
  const uint32_t t = d.tp_size;
  if (d.encoding != ULLM_CUDA_ENCODING_AQ4 && d.encoding != ULLM_CUDA_ENCODING_FP8_CHANNEL)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "stack encoding must be AQ4 or FP8_CHANNEL");
  if (d.layers == 0 || d.hidden == 0 || d.q_heads == 0 || d.kv_heads == 0 || d.head_dim == 0 || d.ffn == 0 ||
      d.vocab == 0 || d.max_tokens == 0 || t == 0)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "stack descriptor has a zero extent");
  if (d.tp_rank >= t) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "tp_rank must be below tp_size");
  if (d.q_heads % t || d.kv_heads % t || d.ffn % t || d.vocab % t)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "q_heads, kv_heads, ffn and vocab must divide by tp_size");
  Comm *cm = nullptr;
  if (t > 1) {
    cm = as_comm(comm);
    if (cm == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "tp_size > 1 needs a live comm");
    if (comm_size(cm) != t || comm_rank(cm) != d.tp_rank)
      return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "comm rank/size differ from the descriptor");
  }
  const uint64_t hd = d.head_dim, qd = uint64_t(d.q_heads) * hd, kvd = uint64_t(d.kv_heads) * hd;
  const uint64_t ql = qd / t, kvl = kvd / t, fl = uint64_t(d.ffn) / t, vl = uint64_t(d.vocab) / t;
  const uint64_t kalign = d.encoding == ULLM_CUDA_ENCODING_AQ4 ? 128 : 16;
  if (d.hidden % kalign || ql % kalign || fl % kalign)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED,
                       "every per-rank K (hidden, q_heads*head_dim/tp, ffn/tp) must be a multiple of 128 (AQ4) or 16 (FP8)");
  if ((ql + 2 * kvl) % 8 || (2 * fl) % 8 || vl % 2 || d.hidden % 8)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "per-rank row lengths must keep rows 16-byte aligned");

  Stack *S = new (std::nothrow) Stack();
  if (S == nullptr) return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  S->ctx = ctx;
  S->queue = q;
  S->stream = q->stream;
  S->comm = cm;
  S->desc = d;
  if (!(S->desc.rms_eps > 0.0f)) S->desc.rms_eps = 1e-5f;

  // ---- plan linears, weight offsets and activation offsets -------------------
  const uint64_t mt = d.max_tokens;
  const uint64_t nq = ql + 2 * kvl;
  uint64_t aoff = 0;
  auto take_act = [&](uint64_t bytes) {
    const uint64_t o = aoff;
    aoff = align_up(aoff + bytes, 256);
    return o;
  };
  S->h0_off = take_act(mt * d.hidden * 4);
  // One set of activation spans shared by all layers, or one set per layer when the
  // caller wants to read every intermediate back (parity checks).
  const uint32_t act_sets = (d.flags & ULLM_CUDA_STACK_FLAG_KEEP_ACTIVATIONS) ? d.layers : 1;
  std::vector<uint64_t> act_qkv_v(act_sets), act_h1_v(act_sets), act_gu_v(act_sets), act_h2_v(act_sets);
  for (uint32_t i = 0; i < act_sets; ++i) {
    act_qkv_v[i] = take_act(mt * nq * 2);
    act_h1_v[i] = take_act(mt * d.hidden * 4);  // h after the attention output projection
    act_gu_v[i] = take_act(mt * fl * 2);
    act_h2_v[i] = take_act(mt * d.hidden * 4);  // h after the MLP
  }
  uint64_t woff = 0;
  auto add = [&](uint32_t layer, uint32_t which, uint64_t full_n, uint64_t full_k, uint64_t n, uint64_t k,
                 uint64_t row_begin, uint64_t col_begin, bool row_parallel) -> StackLinear & {
    StackLinear L;
    L.layer = layer;
    L.which = which;
    L.tensor_id = (uint64_t(layer) << 8) | which | (1ull << 40);
    L.full_n = full_n;
    L.full_k = full_k;
    L.n = n;
    L.k = k;
    L.row_begin = row_begin;
    L.col_begin = col_begin;
    L.row_parallel = row_parallel;
    L.values_off = woff;
    woff = align_up(woff + values_bytes(d.encoding, n, k), 256);
    L.scales_off = woff;
    woff = align_up(woff + scales_bytes(d.encoding, n, k), 256);
    if (!row_parallel) {  // the column-parallel linears start with an RMSNorm: its weight vector
      L.has_norm = true;
      L.norm_tensor_id = (uint64_t(layer) << 8) | which | (2ull << 40);
      L.norm_off = woff;
      woff = align_up(woff + k * 2, 256);
    }
    S->weight_bytes += values_bytes(d.encoding, n, k) + scales_bytes(d.encoding, n, k);
    S->linears.push_back(L);
    return S->linears.back();
  };
  for (uint32_t l = 0; l < d.layers; ++l) {
    const uint32_t si = act_sets == 1 ? 0 : l, sp = act_sets == 1 ? 0 : (l == 0 ? 0 : l - 1);
    const uint64_t act_qkv = act_qkv_v[si], act_h1 = act_h1_v[si], act_gu = act_gu_v[si], act_h2 = act_h2_v[si];
    const uint64_t h_prev = l == 0 ? S->h0_off : act_h2_v[sp];
    {
      StackLinear &L = add(l, ULLM_CUDA_STACK_LINEAR_QKV, qd + 2 * kvd, d.hidden, nq, d.hidden, d.tp_rank * ql, 0, false);
      L.prologue = ULLM_CUDA_PROLOGUE_RMSNORM;
      L.in_off = h_prev;
      L.x_dtype = ULLM_CUDA_DTYPE_F32;
      L.x_stride = d.hidden;
      L.out_off = act_qkv;
      L.y_dtype = ULLM_CUDA_DTYPE_BF16;
      L.y_stride = nq;
    }
    {
      StackLinear &L = add(l, ULLM_CUDA_STACK_LINEAR_O, d.hidden, qd, d.hidden, ql, 0, d.tp_rank * ql, true);
      L.prologue = ULLM_CUDA_PROLOGUE_NONE;
      L.in_off = act_qkv;
      L.x_dtype = ULLM_CUDA_DTYPE_BF16;
      L.x_stride = nq;
      L.has_residual = true;
      L.res_off = h_prev;
      L.out_off = act_h1;
      L.y_dtype = ULLM_CUDA_DTYPE_F32;
      L.y_stride = d.hidden;
    }
    {
      StackLinear &L = add(l, ULLM_CUDA_STACK_LINEAR_GATE_UP, 2ull * d.ffn, d.hidden, 2 * fl, d.hidden, d.tp_rank * fl, 0, false);
      L.prologue = ULLM_CUDA_PROLOGUE_RMSNORM;
      L.epilogue = ULLM_CUDA_EPILOGUE_SWIGLU;  // writes silu(gate) * up: [m, ffn/tp]
      L.in_off = act_h1;
      L.x_dtype = ULLM_CUDA_DTYPE_F32;
      L.x_stride = d.hidden;
      L.out_off = act_gu;
      L.y_dtype = ULLM_CUDA_DTYPE_BF16;
      L.y_stride = fl;
    }
    {
      StackLinear &L = add(l, ULLM_CUDA_STACK_LINEAR_DOWN, d.hidden, d.ffn, d.hidden, fl, 0, d.tp_rank * fl, true);
      L.prologue = ULLM_CUDA_PROLOGUE_NONE;
      L.in_off = act_gu;
      L.x_dtype = ULLM_CUDA_DTYPE_BF16;
      L.x_stride = fl;
      L.has_residual = true;
      L.res_off = act_h1;
      L.out_off = act_h2;
      L.y_dtype = ULLM_CUDA_DTYPE_F32;
      L.y_stride = d.hidden;
    }
  }
  {
    StackLinear &L = add(0, ULLM_CUDA_STACK_LINEAR_LM_HEAD, d.vocab, d.hidden, vl, d.hidden, d.tp_rank * vl, 0, false);
    L.prologue = ULLM_CUDA_PROLOGUE_RMSNORM;
    L.in_off = act_h2_v[act_sets - 1];
    L.x_dtype = ULLM_CUDA_DTYPE_F32;
    L.x_stride = d.hidden;
    L.out_is_step_output = true;
    L.y_dtype = ULLM_CUDA_DTYPE_BF16;
    L.y_stride = vl;
  }

  // ---- allocate ----------------------------------------------------------------
  cudaError_t e = cudaSuccess;
  S->weights = make_buffer(ctx, woff, &e);
  if (S->weights) S->acts = make_buffer(ctx, aoff, &e);
  S->io_out_off = align_up(mt * d.hidden * 2, 256);
  if (S->acts) S->io = make_buffer(ctx, S->io_out_off + align_up(mt * vl * 2, 256), &e);
  if (S->io) e = cudaHostAlloc(&S->pinned_in, mt * d.hidden * 2, cudaHostAllocDefault);
  if (e == cudaSuccess && S->io) e = cudaHostAlloc(&S->pinned_out, mt * vl * 2, cudaHostAllocDefault);
  if (e == cudaSuccess && S->io) e = cudaEventCreateWithFlags(&S->done, cudaEventDisableTiming);
  if (e != cudaSuccess || !S->io) {
    (void)cudaGetLastError();
    (void)destroy_stack(S, false);
    return cuda_error(sink, e, "stack allocation");
  }
  (void)cudaMemsetAsync(S->acts->ptr, 0, aoff, q->stream);
  (void)cudaMemsetAsync(S->io->ptr, 0, S->io->size, q->stream);

  // ---- symmetric peer memory for the fused all-reduce (collective: every rank gets here) --------
  if (t > 1 && !(d.flags & ULLM_CUDA_STACK_FLAG_NCCL_ONLY)) {
    const uint64_t mt8 = mt < 8 ? mt : 8;  // only steps of up to 8 tokens use it
    S->slot_stride = align_up(mt8 * d.hidden * 8, 256);  // {value, tag} pairs
    S->sites = 2 * d.layers;
    uint64_t off = 0;
    for (uint32_t r = 0; r < Stack::kRing; ++r) {
      for (int par = 0; par < 2; ++par) {
        S->ring_slot_off[r][par] = off;
        off += S->slot_stride * t;
      }
    }
    S->step_counter_off = off;
    off += 256;
    std::string why;
    S->push = comm_sym_setup(cm, off, &why);  // false: stay on NCCL (same verdict on every rank)
    // how the consumers gather: per cluster of eight blocks (every block reading every rank's slots costs
    // tp x 64 KiB of L2 reads per block and row; measured per step of the 70B stack, per block / per cluster:
    // 8.75 / 8.11 ms at two ranks, 6.22 / 5.13 ms at four), unless the caller forces one way
    S->gather_cluster = 8u;
    if (d.flags & ULLM_CUDA_STACK_FLAG_GATHER_PER_CLUSTER) S->gather_cluster = 8u;
    if (d.flags & ULLM_CUDA_STACK_FLAG_GATHER_PER_BLOCK) S->gather_cluster = 0u;
#ifdef ULLM_CUDA_TUNING
    if (const char *e = std::getenv("ULLM_CUDA_STACK_CLUSTER")) S->gather_cluster = (uint32_t)std::atoi(e);  // 0, 2, 4, 8
#endif
  }

  // ---- reserve the GEMM path's scratch for the largest step (it cannot grow during capture) ----
  if (d.max_tokens > 1) {
    size_t need = 0;
    // the need is not monotone in the token count (narrow tiles split K more ways): try every tile width
    for (const StackLinear &L : S->linears) {
      for (uint32_t m = 16; ; m *= 2) {
        const uint32_t tokens = m < d.max_tokens ? m : d.max_tokens;
        const size_t b = gemm_scratch_bytes(ctx, make_args(S, L, tokens));
        need = b > need ? b : need;
        if (tokens == d.max_tokens) break;
      }
    }
    e = gemm_reserve_scratch(&q->scratch, need);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      (void)destroy_stack(S, false);
      return cuda_error(sink, e, "stack scratch allocation");
    }
  }

  // ---- generate + quantise the weights --------------------------------------------
  const uint64_t scratch_elems = uint64_t(64) << 20;
  float *scratch = nullptr;
  uint8_t *codes = nullptr;
  e = cudaMalloc(reinterpret_cast<void **>(&scratch), scratch_elems * 4);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&codes), scratch_elems);
  for (size_t i = 0; e == cudaSuccess && i < S->linears.size(); ++i) {
    const StackLinear &L = S->linears[i];
    std::vector<std::pair<uint64_t, uint64_t>> pieces;
    if (L.which == ULLM_CUDA_STACK_LINEAR_QKV) {
      pieces.push_back({d.tp_rank * ql, ql});                  // this rank's query heads
      pieces.push_back({qd + d.tp_rank * kvl, kvl});           // its key heads
      pieces.push_back({qd + kvd + d.tp_rank * kvl, kvl});     // its value heads
    } else if (L.which == ULLM_CUDA_STACK_LINEAR_GATE_UP) {
      pieces.push_back({d.tp_rank * fl, fl});                  // gate rows
      pieces.push_back({uint64_t(d.ffn) + d.tp_rank * fl, fl});  // up rows
    } else {
      pieces.push_back({L.row_begin, L.n});
    }
    e = build_weight(S, L, pieces, scratch, codes, scratch_elems);
    if (e == cudaSuccess && L.has_norm) {  // gamma = bf16(1 + z / 8), the same vector on every rank
      launch_synth_weights(q->stream, d.seed, L.norm_tensor_id, 0, L.k, 1.0f, scratch);
      gamma_kernel<<<(unsigned)((L.k + 255) / 256), 256, 0, q->stream>>>(
          scratch, reinterpret_cast<__nv_bfloat16 *>(static_cast<uint8_t *>(S->weights->ptr) + L.norm_off), L.k);
      e = cudaGetLastError();
      if (e == cudaSuccess) e = cudaStreamSynchronize(q->stream);
    }
  }
  if (scratch) (void)cudaFree(scratch);
  if (codes) (void)cudaFree(codes);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    (void)destroy_stack(S, false);
    return cuda_error(sink, e, "stack weight generation");
  }
  ctx->live_children++;
  registry().add(S);
  *stack = reinterpret_cast<ullm_cuda_stack_t *>(S);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("stack create")
}

ullm_status_t ullm_cuda_stack_step(ullm_cuda_stack_t *stack, uint64_t m, ullm_cuda_tensor_t input_bf16,
                                   ullm_cuda_tensor_t output_bf16, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Stack *S = as_stack(stack);
  if (S == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "stack handle is not live");
  if (m == 0 || m > S->desc.max_tokens) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "m must be in [1, max_tokens]");
  ULLM_CUDA_TRY(cudaSetDevice(S->ctx->device), "cudaSetDevice");
  const uint64_t vl = S->desc.vocab / S->desc.tp_size;
  const uint64_t in_bytes = m * S->desc.hidden * 2, out_bytes = m * vl * 2;
  void *in = nullptr, *out = nullptr;
  st = resolve(input_bf16, in_bytes, 16, S->ctx, "stack input", sink, &in);
  if (st != ULLM_STATUS_OK) return st;
  st = resolve(output_bf16, out_bytes, 16, S->ctx, "stack output", sink, &out);
  if (st != ULLM_STATUS_OK) return st;
  cudaStream_t s = S->queue->stream;
  uint8_t *io = static_cast<uint8_t *>(S->io->ptr);
  ULLM_CUDA_TRY(cudaMemcpyAsync(io, in, in_bytes, cudaMemcpyDeviceToDevice, s), "stack input copy");
  st = run_step(S, static_cast<uint32_t>(m), sink);
  if (st != ULLM_STATUS_OK) return st;
  ULLM_CUDA_TRY(cudaMemcpyAsync(out, io + S->io_out_off, out_bytes, cudaMemcpyDeviceToDevice, s), "stack output copy");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("stack step")
}

ullm_status_t ullm_cuda_stack_step_host(ullm_cuda_stack_t *stack, uint64_t m, const void *host_input_bf16,
                                        void *host_output_bf16, uint32_t timeout_ms,
                                        ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Stack *S = as_stack(stack);
  if (S == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "stack handle is not live");
  if (m == 0 || m > S->desc.max_tokens) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "m must be in [1, max_tokens]");
  if (host_input_bf16 == nullptr || host_output_bf16 == nullptr)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "host pointer is null");
  ULLM_CUDA_TRY(cudaSetDevice(S->ctx->device), "cudaSetDevice");
  const uint64_t vl = S->desc.vocab / S->desc.tp_size;
  const uint64_t in_bytes = m * S->desc.hidden * 2, out_bytes = m * vl * 2;
  cudaStream_t s = S->queue->stream;
  uint8_t *io = static_cast<uint8_t *>(S->io->ptr);
  std::memcpy(S->pinned_in, host_input_bf16, in_bytes);
  ULLM_CUDA_TRY(cudaMemcpyAsync(io, S->pinned_in, in_bytes, cudaMemcpyHostToDevice, s), "stack input upload");
  st = run_step(S, static_cast<uint32_t>(m), sink);
  if (st != ULLM_STATUS_OK) return st;
  ULLM_CUDA_TRY(cudaMemcpyAsync(S->pinned_out, io + S->io_out_off, out_bytes, cudaMemcpyDeviceToHost, s),
                "stack output download");
  ULLM_CUDA_TRY(cudaEventRecord(S->done, s), "cudaEventRecord");
  {
    std::lock_guard<std::mutex> g(S->queue->mutex);
    S->queue->copy_count += 2;
  }
  // bounded wait: poll, never block without a deadline
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (uint64_t spins = 0;; ++spins) {
    cudaError_t e = cudaEventQuery(S->done);
    if (e == cudaSuccess) break;
    if (e != cudaErrorNotReady) return cuda_error(sink, e, "cudaEventQuery");
    if (std::chrono::steady_clock::now() >= deadline)
      return write_error(sink, ULLM_STATUS_CUDA_TIMEOUT, "stack step not complete before the deadline");
    if (spins > 20000) std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
  std::memcpy(host_output_bf16, S->pinned_out, out_bytes);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("stack step host")
}

ullm_status_t ullm_cuda_stack_linear_info(ullm_cuda_stack_t *stack, uint32_t layer, uint32_t which,
                                          ullm_cuda_stack_linear_info_t *info,
                                          ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  st = validate_struct(info, sink, "stack linear info");
  if (st != ULLM_STATUS_OK) return st;
  Stack *S = as_stack(stack);
  if (S == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "stack handle is not live");
  if (which > ULLM_CUDA_STACK_LINEAR_LM_HEAD) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "unknown linear id");
  if (which != ULLM_CUDA_STACK_LINEAR_LM_HEAD && layer >= S->desc.layers)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "layer out of range");
  const size_t idx = which == ULLM_CUDA_STACK_LINEAR_LM_HEAD ? S->linears.size() - 1 : size_t(layer) * 4 + which;
  const StackLinear &L = S->linears[idx];
  info->weight.encoding = S->desc.encoding;
  info->weight.group_size = S->desc.encoding == ULLM_CUDA_ENCODING_AQ4 ? ULLM_CUDA_AQ4_GROUP : 0;
  info->weight.n = L.n;
  info->weight.k = L.k;
  info->weight.values.buffer = reinterpret_cast<ullm_cuda_buffer_t *>(S->weights);
  info->weight.values.offset_bytes = L.values_off;
  info->weight.scales.buffer = reinterpret_cast<ullm_cuda_buffer_t *>(S->weights);
  info->weight.scales.offset_bytes = L.scales_off;
  info->tensor_id = L.tensor_id;
  info->full_n = L.full_n;
  info->full_k = L.full_k;
  info->row_begin = L.row_begin;
  info->col_begin = L.col_begin;
  info->last_input.buffer = reinterpret_cast<ullm_cuda_buffer_t *>(S->acts);
  info->last_input.offset_bytes = L.in_off;
  info->last_output.buffer = reinterpret_cast<ullm_cuda_buffer_t *>(L.out_is_step_output ? S->io : S->acts);
  info->last_output.offset_bytes = L.out_is_step_output ? S->io_out_off : L.out_off;
  info->input_dtype = L.x_dtype;
  info->output_dtype = L.y_dtype;
  info->prologue = L.prologue;
  info->epilogue = L.epilogue;
  info->norm_weight.buffer = L.has_norm ? reinterpret_cast<ullm_cuda_buffer_t *>(S->weights) : nullptr;
  info->norm_weight.offset_bytes = L.has_norm ? L.norm_off : 0;
  info->norm_tensor_id = L.has_norm ? L.norm_tensor_id : 0;
  info->last_residual.buffer = L.has_residual ? reinterpret_cast<ullm_cuda_buffer_t *>(S->acts) : nullptr;
  info->last_residual.offset_bytes = L.has_residual ? L.res_off : 0;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("stack linear info")
}

ullm_status_t ullm_cuda_stack_stats(ullm_cuda_stack_t *stack, uint64_t *weight_bytes, uint64_t *launches_per_step,
                                    ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Stack *S = as_stack(stack);
  if (S == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "stack handle is not live");
  if (weight_bytes) *weight_bytes = S->weight_bytes;
  if (launches_per_step) *launches_per_step = S->launches_per_step;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("stack stats")
}

ullm_status_t ullm_cuda_stack_destroy(ullm_cuda_stack_t **stack, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (stack == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "stack pointer is null");
  Stack *S = as_stack(*stack);
  if (S == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "stack handle is not live");
  registry().remove(S);
  const bool watched = destroy_stack(S, true);
  *stack = nullptr;
  if (!watched)
    return write_error(sink, ULLM_STATUS_CUDA_RUNTIME_ERROR,
                       "stack retired without proof of completion: its memory is abandoned, not freed");
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("stack destroy")
}

}  // extern "C"

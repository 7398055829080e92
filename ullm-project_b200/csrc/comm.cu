// Tensor-parallel communicator: one NCCL rank per process / GPU, NCCL resolved at
// run time with dlopen so that the library loads (and every non-collective entry
// works) on machines without NCCL.
//
// The reference has no multi-GPU code and no collective call site (multi-GPU is
// outside its MVP: docs/plans/main-plan.md:55, docs/architecture/runtime.md:131-141);
// this is new design: row-parallel linears end in a sum over ranks.
#include "internal.hpp"

#include <dlfcn.h>

#include <vector>

namespace ullm {

namespace {

// Minimal NCCL surface, declared here so that no NCCL header is needed to build.
typedef struct ncclComm *ncclComm_t;
typedef struct {
  char internal[128];
} ncclUniqueId;
typedef int ncclResult_t;
constexpr int kNcclSum = 0, kNcclFloat32 = 7, kNcclBfloat16 = 9;

constexpr int kNcclChar = 0;

struct Nccl {
  void *handle = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GetVersion)(int *) = nullptr;
  std::string error;
};

Nccl &nccl() {
  static Nccl *n = [] {
    Nccl *x = new Nccl();
    // RTLD_NOLOAD first: reuse a copy the host process already loaded (same SONAME).
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *nm : names) {
      x->handle = dlopen(nm, RTLD_NOW | RTLD_NOLOAD);
      if (x->handle) break;
    }
    for (int i = 0; i < 2 && !x->handle; ++i) x->handle = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!x->handle) {
      x->error = std::string("NCCL not found: ") + (dlerror() ? dlerror() : "dlopen failed");
      return x;
    }
#define ULLM_SYM(field, name)                                        \
  x->field = reinterpret_cast<decltype(x->field)>(dlsym(x->handle, name)); \
  if (!x->field) x->error = std::string("NCCL symbol missing: ") + name;
    ULLM_SYM(GetUniqueId, "ncclGetUniqueId")
    ULLM_SYM(CommInitRank, "ncclCommInitRank")
    ULLM_SYM(AllReduce, "ncclAllReduce")
    ULLM_SYM(AllGather, "ncclAllGather")
    ULLM_SYM(CommDestroy, "ncclCommDestroy")
    ULLM_SYM(GetErrorString, "ncclGetErrorString")
    ULLM_SYM(GetVersion, "ncclGetVersion")
#undef ULLM_SYM
    return x;
  }();
  return *n;
}

}  // namespace

struct Comm {
  uint32_t magic = kMagicComm;
  Context *ctx = nullptr;
  ncclComm_t comm = nullptr;
  uint32_t rank = 0, size = 1;
  // Symmetric peer memory (same size and layout on every rank), mapped with CUDA IPC:
  // sym[r] is rank r's buffer as seen from this process; sym[rank] is the local one.
  uint8_t *sym[kMaxPeers] = {};
  size_t sym_bytes = 0;
  bool p2p = false;
  bool sym_in_use = false;  // a live stack pushes through the buffer: a second one must not share its slots
};

Comm *as_comm(const ullm_cuda_comm_t *h) {
  Comm *c = checked<Comm>(h);
  return (c && c->magic == kMagicComm) ? c : nullptr;
}
// Collective over the communicator: every rank allocates `bytes` of zeroed device memory and
// maps every peer's allocation (CUDA IPC, peer access over NVLink).  Returns false (and leaves
// the communicator on NCCL only) when any step is not available.
bool comm_sym_setup(Comm *c, size_t bytes, std::string *why) {
  Nccl &n = nccl();
  if (c->sym_in_use) {  // every rank creates and destroys its stacks in the same order: the same verdict everywhere
    if (why) *why = "another stack is using the communicator's symmetric memory";
    return false;
  }
  if (c->p2p && c->sym_bytes >= bytes) {
    // Reuse by a later stack: the slots still hold the previous stack's {value, tag} pairs and step counter.
    // Every rank zeroes its buffer, and one collective makes sure all have done so before anyone pushes again.
    uint8_t *tok = nullptr;
    bool ok = cudaMemset(c->sym[c->rank], 0, c->sym_bytes) == cudaSuccess;
    ok = cudaMalloc(reinterpret_cast<void **>(&tok), 16 * c->size) == cudaSuccess && ok;
    if (tok != nullptr) {
      ok = cudaMemset(tok, 0, 16 * c->size) == cudaSuccess && ok;
      ok = n.AllGather(tok + 16 * c->rank, tok, 16, kNcclChar, c->comm, nullptr) == 0 && ok;
      ok = cudaStreamSynchronize(nullptr) == cudaSuccess && ok;
      (void)cudaFree(tok);
    }
    if (!ok) (void)cudaGetLastError();
    c->sym_in_use = ok;
    return ok;
  }
  if (c->sym_bytes != 0 || c->size > (uint32_t)kMaxPeers) {
    if (why) *why = "symmetric memory already set up with a smaller size, or more ranks than peer slots";
    return false;
  }
  // Every rank walks through the same two all-gathers whatever happens locally, so that no rank
  // is left waiting in a collective and all ranks reach the same verdict.
  uint8_t *local = nullptr;
  uint8_t *hbuf = nullptr;  // [size] IPC handles, then [size] verdict bytes
  const size_t hsz = sizeof(cudaIpcMemHandle_t);
  if (cudaMalloc(reinterpret_cast<void **>(&hbuf), (hsz + 16) * c->size) != cudaSuccess) {
    (void)cudaGetLastError();
    if (why) *why = "device allocation failed";
    return false;
  }
  uint8_t *vbuf = hbuf + hsz * c->size;
  cudaIpcMemHandle_t mine;
  std::memset(&mine, 0, sizeof(mine));
  std::vector<cudaIpcMemHandle_t> all(c->size);
  bool ok = cudaMalloc(reinterpret_cast<void **>(&local), bytes) == cudaSuccess;
  ok = ok && cudaMemset(local, 0, bytes) == cudaSuccess;
  ok = ok && cudaIpcGetMemHandle(&mine, local) == cudaSuccess;
  if (!ok) std::memset(&mine, 0, sizeof(mine));
  bool coll = cudaMemcpy(hbuf + hsz * c->rank, &mine, hsz, cudaMemcpyHostToDevice) == cudaSuccess;
  coll = n.AllGather(hbuf + hsz * c->rank, hbuf, hsz, kNcclChar, c->comm, nullptr) == 0 && coll;
  coll = cudaStreamSynchronize(nullptr) == cudaSuccess && coll;
  coll = cudaMemcpy(all.data(), hbuf, hsz * c->size, cudaMemcpyDeviceToHost) == cudaSuccess && coll;
  ok = ok && coll;
  if (ok) {
    c->sym[c->rank] = local;
    for (uint32_t r = 0; r < c->size && ok; ++r) {
      if (r == c->rank) continue;
      bool zero = true;
      for (size_t i = 0; i < hsz; ++i) zero = zero && reinterpret_cast<const uint8_t *>(&all[r])[i] == 0;
      void *p = nullptr;
      ok = !zero && cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
      c->sym[r] = static_cast<uint8_t *>(p);
    }
  }
  // second round: one verdict byte per rank; peer memory is used only if every rank succeeded
  std::vector<uint8_t> verdict(16 * c->size, 0);
  const uint8_t my_verdict[16] = {static_cast<uint8_t>(ok ? 1 : 0)};
  coll = cudaMemcpy(vbuf + 16 * c->rank, my_verdict, 16, cudaMemcpyHostToDevice) == cudaSuccess;
  coll = n.AllGather(vbuf + 16 * c->rank, vbuf, 16, kNcclChar, c->comm, nullptr) == 0 && coll;
  coll = cudaStreamSynchronize(nullptr) == cudaSuccess && coll;
  coll = cudaMemcpy(verdict.data(), vbuf, 16 * c->size, cudaMemcpyDeviceToHost) == cudaSuccess && coll;
  ok = ok && coll;
  for (uint32_t r = 0; r < c->size; ++r) ok = ok && verdict[16 * r] == 1;
  (void)cudaFree(hbuf);
  if (!ok) {
    (void)cudaGetLastError();
    for (uint32_t r = 0; r < c->size; ++r)
      if (r != c->rank && c->sym[r]) (void)cudaIpcCloseMemHandle(c->sym[r]);
    if (local) (void)cudaFree(local);
    for (auto &q : c->sym) q = nullptr;
    if (why) *why = "CUDA IPC peer mapping is not available on every rank";
    return false;
  }
  c->sym_bytes = bytes;
  c->p2p = true;
  c->sym_in_use = true;
  return true;
}
void comm_sym_release(Comm *c) { c->sym_in_use = false; }
bool comm_p2p(const Comm *c) { return c->p2p; }
uint8_t *comm_sym_ptr(const Comm *c, uint32_t peer) { return c->sym[peer]; }
size_t comm_sym_bytes(const Comm *c) { return c->sym_bytes; }

uint32_t comm_size(const Comm *c) { return c->size; }
uint32_t comm_rank(const Comm *c) { return c->rank; }

cudaError_t comm_all_reduce_raw(Comm *c, cudaStream_t s, void *data, uint64_t count, uint32_t dtype,
                                std::string *why) {
  Nccl &n = nccl();
  const int dt = dtype == ULLM_CUDA_DTYPE_F32 ? kNcclFloat32 : kNcclBfloat16;
  const ncclResult_t r = n.AllReduce(data, data, static_cast<size_t>(count), dt, kNcclSum, c->comm, s);
  if (r != 0) {
    if (why) *why = n.GetErrorString ? n.GetErrorString(r) : "ncclAllReduce failed";
    return cudaErrorUnknown;
  }
  return cudaSuccess;
}

}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_comm_unique_id(uint8_t id[ULLM_CUDA_COMM_ID_BYTES], ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (id == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "id output is null");
  Nccl &n = nccl();
  if (!n.error.empty()) return write_error(sink, ULLM_STATUS_CUDA_COMM_ERROR, n.error.c_str());
  ncclUniqueId u;
  const ncclResult_t r = n.GetUniqueId(&u);
  if (r != 0) return errorf(sink, ULLM_STATUS_CUDA_COMM_ERROR, "ncclGetUniqueId: %s", n.GetErrorString(r));
  std::memcpy(id, u.internal, ULLM_CUDA_COMM_ID_BYTES);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("comm unique id")
}

ullm_status_t ullm_cuda_comm_create(ullm_cuda_context_t *context, const uint8_t id[ULLM_CUDA_COMM_ID_BYTES],
                                    uint32_t rank, uint32_t size, ullm_cuda_comm_t **comm,
                                    ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (comm == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "comm output is null");
  *comm = nullptr;
  Context *c = as_context(context);
  if (c == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "context handle is not live");
  if (id == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "id is null");
  if (size == 0 || size > 64 || rank >= size)
    return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "rank/size out of range");
  Nccl &n = nccl();
  if (!n.error.empty()) return write_error(sink, ULLM_STATUS_CUDA_COMM_ERROR, n.error.c_str());
  ULLM_CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
  ncclUniqueId u;
  std::memcpy(u.internal, id, ULLM_CUDA_COMM_ID_BYTES);
  ncclComm_t nc = nullptr;
  const ncclResult_t r = n.CommInitRank(&nc, static_cast<int>(size), u, static_cast<int>(rank));
  if (r != 0) return errorf(sink, ULLM_STATUS_CUDA_COMM_ERROR, "ncclCommInitRank: %s", n.GetErrorString(r));
  Comm *cm = new (std::nothrow) Comm();
  if (cm == nullptr) {
    n.CommDestroy(nc);
    return write_error(sink, ULLM_STATUS_INTERNAL_ERROR, "host allocation failed");
  }
  cm->ctx = c;
  cm->comm = nc;
  cm->rank = rank;
  cm->size = size;
  c->live_children++;
  registry().add(cm);
  *comm = reinterpret_cast<ullm_cuda_comm_t *>(cm);
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("comm create")
}

ullm_status_t ullm_cuda_comm_all_reduce(ullm_cuda_comm_t *comm, ullm_cuda_queue_t *queue,
                                        ullm_cuda_tensor_t data, uint64_t count, uint32_t dtype,
                                        ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Comm *cm = as_comm(comm);
  if (cm == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "comm handle is not live");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (q->ctx != cm->ctx) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "queue and comm use different contexts");
  if (dtype != ULLM_CUDA_DTYPE_F32 && dtype != ULLM_CUDA_DTYPE_BF16)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "all-reduce dtype must be F32 or BF16");
  if (count == 0) return ULLM_STATUS_OK;
  void *d = nullptr;
  st = resolve(data, count * dtype_bytes(dtype), 16, q->ctx, "all-reduce data", sink, &d);
  if (st != ULLM_STATUS_OK) return st;
  std::string why;
  if (comm_all_reduce_raw(cm, q->stream, d, count, dtype, &why) != cudaSuccess)
    return errorf(sink, ULLM_STATUS_CUDA_COMM_ERROR, "ncclAllReduce: %s", why.c_str());
  std::lock_guard<std::mutex> g(q->mutex);
  q->dispatch_count += 1;
  q->total_dispatch += 1;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("comm all reduce")
}

ullm_status_t ullm_cuda_comm_destroy(ullm_cuda_comm_t **comm, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (comm == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "comm pointer is null");
  Comm *cm = as_comm(*comm);
  if (cm == nullptr) return write_error(sink, ULLM_STATUS_CUDA_INVALID_HANDLE, "comm handle is not live");
  registry().remove(cm);
  (void)cudaSetDevice(cm->ctx->device);
  // Destroying a communicator is collective and NCCL's own teardown waits for its kernels; the peers'
  // mappings are closed first, which needs every stack that pushed through them to be gone (it is: a stack
  // counts as a child of the context until its queue's work has been observed complete).
  for (uint32_t r = 0; r < cm->size && r < (uint32_t)kMaxPeers; ++r) {
    if (cm->sym[r] == nullptr) continue;
    if (r == cm->rank)
      (void)cudaFree(cm->sym[r]);
    else
      (void)cudaIpcCloseMemHandle(cm->sym[r]);
  }
  nccl().CommDestroy(cm->comm);
  cm->ctx->live_children--;
  cm->magic = 0;
  delete cm;
  *comm = nullptr;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("comm destroy")
}

}  // extern "C"

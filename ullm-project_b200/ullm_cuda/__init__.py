"""Safe host-side access to the CUDA backend's C ABI.

Python stand-in for the `ullm-cuda` crate, shaped after the reference's safe HIP
wrapper (crates/ullm-hip/src/lib.rs): `Status` with `from_raw` / `raw`
(:20-76), an error type carrying status + native diagnostic (:78-110),
`abi_version()`, `version()`, `backend_probe()`, `context_probe()` (:189-268),
and submit -> wait -> drop completions (:293-441).  Unlike the reference's
Phase-1 wrapper this backend executes numerical work — on the GPU only.
Nothing in this package computes on the CPU; a missing library or device is an
error, never a fallback.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from enum import Enum

import numpy as np

from . import _abi as abi
from ._abi import (EPILOGUE_NONE, EPILOGUE_SWIGLU, DTYPE_BF16, DTYPE_F16, DTYPE_F32, DTYPE_F8E4M3FN, DTYPE_I8, DTYPE_U8, ENCODING_AQ4,  # noqa: F401
                   ENCODING_FP8_CHANNEL, ENCODING_NVFP4, KERNEL_AUTO, KERNEL_GEMM, KERNEL_MATVEC, LINEAR_DOWN,
                   LINEAR_GATE_UP, LINEAR_LM_HEAD, LINEAR_O, LINEAR_QKV, PROLOGUE_NONE, PROLOGUE_RMSNORM,
                   PROLOGUE_SWIGLU, STACK_FLAG_GATHER_PER_BLOCK, STACK_FLAG_GATHER_PER_CLUSTER,
                   STACK_FLAG_KEEP_ACTIVATIONS, STACK_FLAG_NCCL_ONLY, STACK_FLAG_NO_GRAPH)

ERROR_CAPACITY = 512


class Status(Enum):
    Ok = 0
    InvalidArgument = 1
    BufferTooSmall = 2
    Unsupported = 3
    CudaUnavailable = 4
    InvalidAbiVersion = 5
    ReservedNonzero = 6
    InternalError = 7
    Timeout = 8
    InvalidHandle = 9
    ZeroDispatch = 10
    RuntimeError = 11
    DispatchContract = 12
    OutOfMemory = 13
    OutOfRange = 14
    CommError = 15
    DeviceFlagged = 16
    Unknown = -1

    @classmethod
    def from_raw(cls, raw: int) -> "Status":
        try:
            return cls(int(raw)) if int(raw) >= 0 else cls.Unknown
        except ValueError:
            return cls.Unknown


class CudaError(Exception):
    """A non-OK status from the native library, with its diagnostic."""

    def __init__(self, status: Status, message: str, raw: int | None = None):
        super().__init__(f"{status.name}: {message}")
        self.status = status
        self.message = message
        self.raw = status.value if raw is None else raw


def _sink(capacity: int = ERROR_CAPACITY):
    buf = C.create_string_buffer(capacity)
    s = abi.ErrorSink()
    s.struct_size = C.sizeof(abi.ErrorSink)
    s.abi_version = abi.ABI_VERSION
    s.message = C.cast(buf, C.c_void_p)
    s.message_capacity = capacity
    return s, buf


def _check(raw: int, sink, buf):
    if raw != abi.OK:
        raise CudaError(Status.from_raw(raw), buf.value.decode("utf-8", "replace"), raw)


def _call(name: str, *args):
    s, buf = _sink()
    raw = getattr(abi.load(), name)(*args, C.byref(s))
    _check(raw, s, buf)


@dataclass(frozen=True)
class Version:
    abi_version: int
    major: int
    minor: int
    patch: int


@dataclass(frozen=True)
class BackendProbe:
    backend: int
    available: bool
    cuda_runtime_present: bool
    device_count: int
    sm: tuple
    sm_count: int
    l2_mib: int
    global_memory_bytes: int
    diagnostic: str


def abi_version() -> int:
    v = C.c_uint32(0)
    _call("ullm_cuda_get_abi_version", C.byref(v))
    return v.value


def version() -> Version:
    info = abi.VersionInfo(struct_size=C.sizeof(abi.VersionInfo), abi_version=abi.ABI_VERSION)
    _call("ullm_cuda_query_version", C.byref(info))
    return Version(abi_version(), info.major, info.minor, info.patch)


def backend_probe() -> BackendProbe:
    """`CudaUnavailable` is a result here, not a failure (crates/ullm-hip/src/lib.rs:230-242)."""
    r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult), abi_version=abi.ABI_VERSION)
    s, buf = _sink()
    raw = abi.load().ullm_cuda_backend_probe(abi.BACKEND_CUDA, C.byref(r), C.byref(s))
    if raw not in (abi.OK, abi.CUDA_UNAVAILABLE):
        _check(raw, s, buf)
    return BackendProbe(r.backend, bool(r.available), bool(r.cuda_runtime_present), r.device_count,
                        (r.sm_major, r.sm_minor), r.sm_count, r.l2_bytes_mib, r.global_memory_bytes,
                        buf.value.decode())


def available() -> bool:
    return backend_probe().available


class _Handle:
    _destroy = None

    def __init__(self):
        self._h = C.c_void_p(None)

    @property
    def handle(self):
        return self._h

    def close(self):
        if self._h and self._h.value:
            _call(self._destroy, C.byref(self._h))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Context(_Handle):
    _destroy = "ullm_cuda_context_destroy"

    def __init__(self, device: int = 0):
        super().__init__()
        _call("ullm_cuda_context_create", device, C.byref(self._h))
        self.device = device

    def probe(self):
        r = abi.ContextProbeResult(struct_size=C.sizeof(abi.ContextProbeResult), abi_version=abi.ABI_VERSION)
        _call("ullm_cuda_context_probe", self._h, C.byref(r))
        return r

    def shutdown(self, timeout_ms: int = 60000) -> int:
        """Refuses new prepares / submits, drains what is in flight; returns how many submissions failed."""
        failed = C.c_uint32(0)
        _call("ullm_cuda_context_shutdown", self._h, int(timeout_ms), C.byref(failed))
        return failed.value

    def set_wait_limit(self, limit_ms: int):
        """Limit of every device-side wait of kernels launched for this context from now on."""
        _call("ullm_cuda_context_set_wait_limit", self._h, int(limit_ms))

    def queue(self) -> "Queue":
        return Queue(self)

    def alloc(self, nbytes: int) -> "Buffer":
        return Buffer(self, nbytes)


class Buffer(_Handle):
    _destroy = "ullm_cuda_buffer_free"

    def __init__(self, ctx: Context, nbytes: int):
        super().__init__()
        _call("ullm_cuda_buffer_alloc", ctx.handle, int(nbytes), C.byref(self._h))
        self.nbytes = int(nbytes)
        self.ctx = ctx

    def at(self, offset: int = 0) -> abi.Tensor:
        return abi.Tensor(self._h, int(offset))


class Completion(_Handle):
    _destroy = "ullm_cuda_completion_destroy"

    def wait(self, timeout_ms: int = 60000) -> abi.CompletionResult:
        """Consumes the handle whatever the outcome, a timeout included (the reference's rule:
        crates/ullm-hip/src/lib.rs:404-441 drops the completion after every wait)."""
        r = abi.CompletionResult(struct_size=C.sizeof(abi.CompletionResult), abi_version=abi.ABI_VERSION)
        s, buf = _sink()
        raw = abi.load().ullm_cuda_completion_wait(self._h, min(int(timeout_ms), 0xFFFFFFFF), C.byref(r), C.byref(s))
        self._h = C.c_void_p(None)
        self.last_result = r
        _check(raw, s, buf)
        return r

    def query(self, timeout_ms: int = 0) -> bool:
        s, buf = _sink()
        raw = abi.load().ullm_cuda_completion_query(self._h, int(timeout_ms), C.byref(s))
        if raw == abi.CUDA_TIMEOUT:
            return False
        _check(raw, s, buf)
        return True

    def elapsed_ms_since(self, start: "Completion") -> float:
        ms = C.c_float(0)
        _call("ullm_cuda_completion_elapsed_ms", start.handle, self._h, C.byref(ms))
        return ms.value


class Graph(_Handle):
    _destroy = "ullm_cuda_graph_destroy"

    def launch(self, queue: "Queue"):
        _call("ullm_cuda_graph_launch", self._h, queue.handle)


class Queue(_Handle):
    _destroy = "ullm_cuda_queue_destroy"

    def __init__(self, ctx: Context):
        super().__init__()
        _call("ullm_cuda_queue_create", ctx.handle, C.byref(self._h))
        self.ctx = ctx

    # -- data movement ---------------------------------------------------------
    def upload(self, dst: abi.Tensor, array: np.ndarray):
        a = np.ascontiguousarray(array)
        _call("ullm_cuda_buffer_upload", self._h, dst, a.ctypes.data_as(C.c_void_p), a.nbytes)

    def download(self, src: abi.Tensor, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        _call("ullm_cuda_buffer_download", self._h, src, out.ctypes.data_as(C.c_void_p), out.nbytes)
        return out

    def fill(self, dst: abi.Tensor, value: int, nbytes: int):
        _call("ullm_cuda_buffer_fill", self._h, dst, value, nbytes)

    def signal(self) -> Completion:
        c = Completion()
        _call("ullm_cuda_queue_signal", self._h, C.byref(c._h))
        return c

    def synchronize(self, timeout_ms: int = 600000) -> abi.CompletionResult:
        return self.signal().wait(timeout_ms)

    # -- graphs ----------------------------------------------------------------
    def capture_begin(self):
        _call("ullm_cuda_queue_capture_begin", self._h)

    def capture_end(self) -> Graph:
        g = Graph()
        _call("ullm_cuda_queue_capture_end", self._h, C.byref(g._h))
        return g

    # -- ops -------------------------------------------------------------------
    def synth_weights(self, seed, tensor_id, first, count, std, out: abi.Tensor):
        _call("ullm_cuda_synth_weights", self._h, seed, tensor_id, first, count, C.c_float(std), out)

    def synth_activations(self, seed, tensor_id, first, count, out: abi.Tensor):
        _call("ullm_cuda_synth_activations", self._h, seed, tensor_id, first, count, out)

    def quantize(self, src_f32: abi.Tensor, weight: abi.Weight):
        _call("ullm_cuda_quantize", self._h, src_f32, C.byref(weight))

    def quantize_safetensors(self, path: str, name: str, weight: abi.Weight):
        """Loads tensor `name` [N, K] of a safetensors file and quantises it on the device into `weight`."""
        _call("ullm_cuda_quantize_safetensors", self._h, path.encode(), name.encode(), C.byref(weight))

    def aq4_unpack(self, weight: abi.Weight, out_i8: abi.Tensor):
        _call("ullm_cuda_aq4_unpack", self._h, C.byref(weight), out_i8)

    def aq4_pack(self, src_i8: abi.Tensor, weight: abi.Weight):
        _call("ullm_cuda_aq4_pack", self._h, src_i8, C.byref(weight))

    def dequantize(self, weight: abi.Weight, out: abi.Tensor, out_dtype: int):
        _call("ullm_cuda_dequantize", self._h, C.byref(weight), out, out_dtype)

    def linear_enqueue(self, desc: abi.LinearDesc):
        _call("ullm_cuda_linear_enqueue", self._h, C.byref(desc))

    def linear_enqueue_static_scratch(self, desc: abi.LinearDesc):
        """The GEMM-path linear without any device allocation: its activation staging area is a fixed
        array inside the library (limits: M*K*2 <= abi.STATIC_SCRATCH_BYTES, no SwiGLU epilogue).
        Calls on one device share that array, so they must not overlap on the GPU."""
        _call("ullm_cuda_linear_enqueue_static_scratch", self._h, C.byref(desc))

    def linear_enqueue_partial(self, desc: abi.LinearDesc, slots: abi.Slots):
        """Producer half of the fused all-reduce: the fp32 results go to slot `slots.rank` as {value, tag} pairs."""
        _call("ullm_cuda_linear_enqueue_partial", self._h, C.byref(desc), C.byref(slots))

    def linear_enqueue_reduced(self, desc: abi.LinearDesc, slots: abi.Slots, reduced_out: abi.Tensor | None = None):
        """Consumer half: the input is bf16(residual + sum of the ranks' slots); `reduced_out` receives that sum."""
        _call("ullm_cuda_linear_enqueue_reduced", self._h, C.byref(desc), C.byref(slots),
              reduced_out if reduced_out is not None else abi.Tensor(None, 0))

    def linear_submit(self, desc: abi.LinearDesc) -> Completion:
        c = Completion()
        _call("ullm_cuda_linear_submit", self._h, C.byref(desc), C.byref(c._h))
        return c


def weight_desc(encoding: int, n: int, k: int, values: abi.Tensor, scales: abi.Tensor) -> abi.Weight:
    group = {ENCODING_AQ4: 128, ENCODING_NVFP4: 16}.get(encoding, 0)
    return abi.Weight(encoding, group, n, k, values, scales)


def weight_bytes(encoding: int, n: int, k: int):
    """(values bytes, scales bytes) of a quantised W[N,K]."""
    if encoding == ENCODING_AQ4:
        return n * (k // 2), n * (k // 128) * 2
    if encoding == ENCODING_NVFP4:  # f16 block scales, then the f32 tensor scale at the next 16-byte boundary
        return n * (k // 2), (n * (k // 16) * 2 + 15) // 16 * 16 + 4
    return n * k, n * 4


def linear_desc(weight: abi.Weight, m: int, x: abi.Tensor, y: abi.Tensor, *, input_dtype=DTYPE_BF16,
                output_dtype=DTYPE_BF16, prologue=PROLOGUE_NONE, kernel=KERNEL_AUTO, rms_eps=1e-5,
                input_row_stride=0, output_row_stride=0, epilogue=EPILOGUE_NONE, norm_weight: abi.Tensor | None = None,
                residual: abi.Tensor | None = None, residual_row_stride=0) -> abi.LinearDesc:
    d = abi.LinearDesc()
    d.struct_size = C.sizeof(abi.LinearDesc)
    d.abi_version = abi.ABI_VERSION
    d.weight = weight
    d.m = m
    d.input = x
    d.input_row_stride = input_row_stride
    d.output = y
    d.output_row_stride = output_row_stride
    d.input_dtype = input_dtype
    d.output_dtype = output_dtype
    d.prologue = prologue
    d.kernel = kernel
    d.rms_eps = rms_eps
    d.epilogue = epilogue
    if norm_weight is not None:
        d.norm_weight = norm_weight
    if residual is not None:
        d.residual = residual
    d.residual_row_stride = residual_row_stride
    return d


def slots_desc(slots: abi.Tensor, rank_stride_bytes: int, ranks: int, *, rank: int = 0, tag: int = 1,
               gather: int = 0) -> abi.Slots:
    s = abi.Slots()
    s.struct_size = C.sizeof(abi.Slots)
    s.abi_version = abi.ABI_VERSION
    s.slots = slots
    s.rank_stride_bytes = rank_stride_bytes
    s.ranks, s.rank, s.tag, s.gather = ranks, rank, tag, gather
    return s


def linear_supports(desc: abi.LinearDesc) -> int:
    """Selected kernel id, or raises CudaError(Unsupported / argument error). No device needed."""
    k = C.c_uint32(0)
    _call("ullm_cuda_linear_supports", C.byref(desc), C.byref(k))
    return k.value


def safetensors_find(path: str, name: str) -> abi.SafetensorsInfo:
    """Dtype, shape and position of one tensor of a safetensors file (header only; no device)."""
    info = abi.SafetensorsInfo(struct_size=C.sizeof(abi.SafetensorsInfo), abi_version=abi.ABI_VERSION)
    _call("ullm_cuda_safetensors_find", path.encode(), name.encode(), C.byref(info))
    return info


def plan_op(encoding: int, m: int, n: int, k: int, *, input_dtype=DTYPE_BF16, output_dtype=DTYPE_BF16, prologue=PROLOGUE_NONE,
            epilogue=EPILOGUE_NONE, kernel=KERNEL_AUTO, rms_eps=1e-5, norm_weight=False, residual=False) -> abi.PlanOp:
    """One quantised linear of a plan: metadata only (the buffers arrive with each submission)."""
    o = abi.PlanOp()
    o.struct_size = C.sizeof(abi.PlanOp)
    o.abi_version = abi.ABI_VERSION
    o.encoding, o.group_size = encoding, 128 if encoding == ENCODING_AQ4 else 0
    o.n, o.k, o.m = n, k, m
    o.input_dtype, o.output_dtype, o.prologue, o.epilogue, o.kernel, o.rms_eps = input_dtype, output_dtype, prologue, epilogue, kernel, rms_eps
    o.flags = (abi.PLAN_OP_HAS_NORM_WEIGHT if norm_weight else 0) | (abi.PLAN_OP_HAS_RESIDUAL if residual else 0)
    return o


def binding(op_index: int, slot: int, access: int, tensor: abi.Tensor) -> abi.Binding:
    b = abi.Binding()
    b.struct_size = C.sizeof(abi.Binding)
    b.abi_version = abi.ABI_VERSION
    b.op_index, b.slot, b.access, b.tensor = op_index, slot, access, tensor
    return b


class Event(_Handle):
    """Completion of one submission.  Never consumed by query or wait; dropping it does not stop the context's
    executor from watching the submission."""
    _destroy = "ullm_cuda_event_destroy"

    def query(self) -> int:
        """abi.EVENT_PENDING / EVENT_SUCCESS; a failed submission raises CudaError with the stored diagnostic."""
        st = C.c_uint32(0)
        _call("ullm_cuda_event_query", self._h, C.byref(st))
        return st.value

    def wait(self, timeout_ms: int = 60000):
        _call("ullm_cuda_event_wait", self._h, int(timeout_ms))


class Prepared(_Handle):
    """A prepared plan: the ops' metadata copied into the library and their kernels chosen."""
    _destroy = "ullm_cuda_prepared_destroy"

    def __init__(self, ctx: "Context", ops):
        super().__init__()
        arr = (abi.PlanOp * len(ops))(*ops)
        _call("ullm_cuda_prepare", ctx.handle, arr, len(ops), C.byref(self._h))

    def submit(self, queue: "Queue", bindings, wait=(), want_event: bool = True):
        arr = (abi.Binding * max(len(bindings), 1))(*bindings)
        deps = (C.c_void_p * max(len(wait), 1))(*[e.handle for e in wait])
        ev = Event()
        _call("ullm_cuda_submit", queue.handle, self._h, arr, len(bindings), deps, len(wait),
              C.byref(ev._h) if want_event else None)
        return ev if want_event else None


class Comm(_Handle):
    _destroy = "ullm_cuda_comm_destroy"

    @staticmethod
    def unique_id() -> bytes:
        raw = (C.c_uint8 * abi.COMM_ID_BYTES)()
        _call("ullm_cuda_comm_unique_id", raw)
        return bytes(raw)

    def __init__(self, ctx: Context, uid: bytes, rank: int, size: int):
        super().__init__()
        raw = (C.c_uint8 * abi.COMM_ID_BYTES).from_buffer_copy(uid)
        _call("ullm_cuda_comm_create", ctx.handle, raw, rank, size, C.byref(self._h))
        self.rank, self.size = rank, size

    def all_reduce(self, queue: Queue, data: abi.Tensor, count: int, dtype: int = DTYPE_F32):
        _call("ullm_cuda_comm_all_reduce", self._h, queue.handle, data, count, dtype)


@dataclass
class StackShape:
    """Shape of a decoder's linear stack (counts of heads, widths)."""
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int

    def weight_elements(self) -> int:
        qkv = (self.q_heads + 2 * self.kv_heads) * self.head_dim * self.hidden
        o = self.hidden * self.q_heads * self.head_dim
        return self.layers * (qkv + o + 3 * self.hidden * self.ffn) + self.vocab * self.hidden


LLAMA3_8B = StackShape(32, 4096, 32, 8, 128, 14336, 128256)
LLAMA3_70B = StackShape(80, 8192, 64, 8, 128, 28672, 128256)


class Stack(_Handle):
    _destroy = "ullm_cuda_stack_destroy"

    def __init__(self, ctx: Context, queue: Queue, shape: StackShape, encoding: int, *, max_tokens: int,
                 seed: int = 20260803, tp_rank: int = 0, tp_size: int = 1, comm: Comm | None = None,
                 flags: int = 0, rms_eps: float = 1e-5):
        super().__init__()
        d = abi.StackDesc()
        d.struct_size = C.sizeof(abi.StackDesc)
        d.abi_version = abi.ABI_VERSION
        d.encoding = encoding
        d.layers, d.hidden, d.q_heads, d.kv_heads = shape.layers, shape.hidden, shape.q_heads, shape.kv_heads
        d.head_dim, d.ffn, d.vocab = shape.head_dim, shape.ffn, shape.vocab
        d.tp_rank, d.tp_size, d.max_tokens, d.flags, d.seed, d.rms_eps = tp_rank, tp_size, max_tokens, flags, seed, rms_eps
        self.desc = d
        self.shape = shape
        self.queue = queue
        _call("ullm_cuda_stack_create", ctx.handle, queue.handle, comm.handle if comm else None, C.byref(d),
              C.byref(self._h))

    @property
    def local_vocab(self) -> int:
        return self.shape.vocab // self.desc.tp_size

    def step(self, m: int, x: abi.Tensor, y: abi.Tensor):
        _call("ullm_cuda_stack_step", self._h, m, x, y)

    def step_host(self, x_bits: np.ndarray, timeout_ms: int = 600000) -> np.ndarray:
        """bf16 bit patterns [m, hidden] in host memory -> logits bits [m, vocab/tp] in host memory."""
        x = np.ascontiguousarray(x_bits, np.uint16)
        m = x.shape[0]
        out = np.empty((m, self.local_vocab), np.uint16)
        _call("ullm_cuda_stack_step_host", self._h, m, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
              timeout_ms)
        return out

    def step_host_into(self, x: np.ndarray, out: np.ndarray, timeout_ms: int = 600000):
        _call("ullm_cuda_stack_step_host", self._h, x.shape[0], x.ctypes.data_as(C.c_void_p),
              out.ctypes.data_as(C.c_void_p), timeout_ms)

    def linear_info(self, layer: int, which: int) -> abi.StackLinearInfo:
        info = abi.StackLinearInfo(struct_size=C.sizeof(abi.StackLinearInfo), abi_version=abi.ABI_VERSION)
        _call("ullm_cuda_stack_linear_info", self._h, layer, which, C.byref(info))
        return info

    def stats(self):
        wb, lp = C.c_uint64(0), C.c_uint64(0)
        _call("ullm_cuda_stack_stats", self._h, C.byref(wb), C.byref(lp))
        return wb.value, lp.value


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)

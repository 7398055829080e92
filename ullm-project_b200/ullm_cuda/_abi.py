"""ctypes declarations of the C ABI in include/ullm_cuda.h (one-to-one).

This is the Python stand-in for the `ullm-cuda-sys` crate: like
crates/ullm-hip-sys/src/bindings.rs:100-119 it only declares the foreign
functions and mirrors the struct layouts; it contains no logic.  The shared
library must exist — there is no fallback of any kind.
"""

from __future__ import annotations

import ctypes as C
import os

ABI_VERSION = 1
BACKEND_CUDA = 2

# status codes (include/ullm_cuda.h)
OK, INVALID_ARGUMENT, BUFFER_TOO_SMALL, UNSUPPORTED, CUDA_UNAVAILABLE = 0, 1, 2, 3, 4
INVALID_ABI_VERSION, RESERVED_NONZERO, INTERNAL_ERROR = 5, 6, 7
CUDA_TIMEOUT, CUDA_INVALID_HANDLE, CUDA_ZERO_DISPATCH, CUDA_RUNTIME_ERROR = 8, 9, 10, 11
CUDA_DISPATCH_CONTRACT, CUDA_OUT_OF_MEMORY, CUDA_OUT_OF_RANGE, CUDA_COMM_ERROR, CUDA_DEVICE_FLAGGED = 12, 13, 14, 15, 16

DTYPE_BF16, DTYPE_F16, DTYPE_F32, DTYPE_F8E4M3FN, DTYPE_I8, DTYPE_U8 = 0, 1, 2, 3, 7, 8
ENCODING_UNQUANTIZED, ENCODING_NVFP4, ENCODING_AQ4, ENCODING_FP8_CHANNEL = 0, 1, 2, 3
PROLOGUE_NONE, PROLOGUE_RMSNORM, PROLOGUE_SWIGLU = 0, 1, 2
EPILOGUE_NONE, EPILOGUE_SWIGLU = 0, 1
KERNEL_AUTO, KERNEL_MATVEC, KERNEL_GEMM = 0, 1, 2
ACCESS_READ, ACCESS_WRITE, ACCESS_READ_WRITE = 1, 2, 3
PLAN_OP_HAS_NORM_WEIGHT, PLAN_OP_HAS_RESIDUAL = 1, 2
SLOT_WEIGHT_VALUES, SLOT_WEIGHT_SCALES, SLOT_INPUT, SLOT_OUTPUT, SLOT_NORM_WEIGHT, SLOT_RESIDUAL = 0, 1, 2, 3, 4, 5
EVENT_PENDING, EVENT_SUCCESS, EVENT_FAILURE = 0, 1, 2
STACK_FLAG_NO_GRAPH = 1
STACK_FLAG_KEEP_ACTIVATIONS = 2
STACK_FLAG_NCCL_ONLY = 4
STACK_FLAG_GATHER_PER_BLOCK = 8
STACK_FLAG_GATHER_PER_CLUSTER = 16
LINEAR_QKV, LINEAR_O, LINEAR_GATE_UP, LINEAR_DOWN, LINEAR_LM_HEAD = 0, 1, 2, 3, 4
COMM_ID_BYTES = 128
STATIC_SCRATCH_BYTES = 8 << 20

u32, u64, vp = C.c_uint32, C.c_uint64, C.c_void_p


class ErrorSink(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("message", C.c_void_p), ("message_capacity", u64),
                ("message_length", u64), ("reserved", u64 * 2)]


class VersionInfo(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("major", u32), ("minor", u32), ("patch", u32),
                ("reserved", u32 * 3)]


class BackendProbeResult(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("backend", u32), ("available", u32),
                ("cuda_runtime_present", u32), ("device_count", u32), ("sm_major", u32), ("sm_minor", u32),
                ("sm_count", u32), ("l2_bytes_mib", u32), ("global_memory_bytes", u64), ("reserved", u32 * 4)]


class ContextProbeResult(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("context_present", u32), ("cuda_available", u32),
                ("device_ordinal", u32), ("reserved", u32 * 3)]


class Tensor(C.Structure):
    _fields_ = [("buffer", vp), ("offset_bytes", u64)]


class Weight(C.Structure):
    _fields_ = [("encoding", u32), ("group_size", u32), ("n", u64), ("k", u64), ("values", Tensor),
                ("scales", Tensor)]


class CompletionResult(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("dispatch_count", u64), ("copy_count", u64),
                ("selected_backend", u32), ("fallback_used", u32), ("terminal", u32), ("device_flags", u32),
                ("reserved", u32 * 4)]


class LinearDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("weight", Weight), ("m", u64), ("input", Tensor),
                ("input_row_stride", u64), ("output", Tensor), ("output_row_stride", u64), ("input_dtype", u32),
                ("output_dtype", u32), ("prologue", u32), ("kernel", u32), ("rms_eps", C.c_float),
                ("epilogue", u32), ("norm_weight", Tensor), ("residual", Tensor), ("residual_row_stride", u64),
                ("reserved", u32 * 4)]


class Slots(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("slots", Tensor), ("rank_stride_bytes", u64),
                ("ranks", u32), ("rank", u32), ("tag", u32), ("gather", u32), ("reserved", u32 * 4)]


class PlanOp(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("encoding", u32), ("group_size", u32), ("n", u64), ("k", u64),
                ("m", u64), ("input_dtype", u32), ("output_dtype", u32), ("prologue", u32), ("epilogue", u32),
                ("kernel", u32), ("flags", u32), ("rms_eps", C.c_float), ("reserved", u32 * 5)]


class Binding(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("op_index", u32), ("slot", u32), ("access", u32),
                ("reserved0", u32), ("tensor", Tensor), ("reserved", u32 * 4)]


class SafetensorsInfo(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("dtype", u32), ("rank", u32), ("rows", u64), ("cols", u64),
                ("data_offset", u64), ("data_bytes", u64), ("reserved", u32 * 4)]


class StackDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("encoding", u32), ("layers", u32), ("hidden", u32),
                ("q_heads", u32), ("kv_heads", u32), ("head_dim", u32), ("ffn", u32), ("vocab", u32),
                ("tp_rank", u32), ("tp_size", u32), ("max_tokens", u32), ("flags", u32), ("seed", u64),
                ("rms_eps", C.c_float), ("reserved", u32 * 5)]


class StackLinearInfo(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("weight", Weight), ("tensor_id", u64), ("full_n", u64),
                ("full_k", u64), ("row_begin", u64), ("col_begin", u64), ("last_input", Tensor),
                ("last_output", Tensor), ("input_dtype", u32), ("output_dtype", u32), ("prologue", u32),
                ("epilogue", u32), ("norm_weight", Tensor), ("last_residual", Tensor), ("norm_tensor_id", u64),
                ("reserved", u32 * 4)]


# sizes pinned in the header's static_asserts
EXPECTED_SIZES = {
    ErrorSink: 48, VersionInfo: 32, BackendProbeResult: 64, ContextProbeResult: 32, Tensor: 16, Weight: 56,
    CompletionResult: 56, LinearDesc: 200, StackDesc: 88, StackLinearInfo: 208, Slots: 64, PlanOp: 88, Binding: 56, SafetensorsInfo: 64,
}

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("ULLM_CUDA_LIB", os.path.join(_PKG, "lib", "libullm_cuda.so"))

P = C.POINTER
SINK = P(ErrorSink)

# name -> argtypes (restype is always ullm_status_t = uint32)
SIGNATURES = {
    "ullm_cuda_get_abi_version": [P(u32), SINK],
    "ullm_cuda_query_version": [P(VersionInfo), SINK],
    "ullm_cuda_backend_probe": [u32, P(BackendProbeResult), SINK],
    "ullm_cuda_context_probe": [vp, P(ContextProbeResult), SINK],
    "ullm_cuda_context_create": [u32, P(vp), SINK],
    "ullm_cuda_context_destroy": [P(vp), SINK],
    "ullm_cuda_context_set_wait_limit": [vp, u32, SINK],
    "ullm_cuda_queue_create": [vp, P(vp), SINK],
    "ullm_cuda_queue_destroy": [P(vp), SINK],
    "ullm_cuda_buffer_alloc": [vp, u64, P(vp), SINK],
    "ullm_cuda_buffer_free": [P(vp), SINK],
    "ullm_cuda_buffer_size": [vp, P(u64), SINK],
    "ullm_cuda_buffer_upload": [vp, Tensor, vp, u64, SINK],
    "ullm_cuda_buffer_download": [vp, Tensor, vp, u64, SINK],
    "ullm_cuda_buffer_fill": [vp, Tensor, C.c_uint8, u64, SINK],
    "ullm_cuda_queue_signal": [vp, P(vp), SINK],
    "ullm_cuda_completion_wait": [vp, u32, P(CompletionResult), SINK],
    "ullm_cuda_completion_elapsed_ms": [vp, vp, P(C.c_float), SINK],
    "ullm_cuda_completion_query": [vp, u32, SINK],
    "ullm_cuda_completion_destroy": [P(vp), SINK],
    "ullm_cuda_queue_capture_begin": [vp, SINK],
    "ullm_cuda_queue_capture_end": [vp, P(vp), SINK],
    "ullm_cuda_graph_launch": [vp, vp, SINK],
    "ullm_cuda_graph_destroy": [P(vp), SINK],
    "ullm_cuda_synth_weights": [vp, u64, u64, u64, u64, C.c_float, Tensor, SINK],
    "ullm_cuda_synth_activations": [vp, u64, u64, u64, u64, Tensor, SINK],
    "ullm_cuda_quantize": [vp, Tensor, P(Weight), SINK],
    "ullm_cuda_aq4_unpack": [vp, P(Weight), Tensor, SINK],
    "ullm_cuda_aq4_pack": [vp, Tensor, P(Weight), SINK],
    "ullm_cuda_dequantize": [vp, P(Weight), Tensor, u32, SINK],
    "ullm_cuda_linear_supports": [P(LinearDesc), P(u32), SINK],
    "ullm_cuda_linear_enqueue": [vp, P(LinearDesc), SINK],
    "ullm_cuda_linear_submit": [vp, P(LinearDesc), P(vp), SINK],
    "ullm_cuda_linear_enqueue_static_scratch": [vp, P(LinearDesc), SINK],
    "ullm_cuda_safetensors_find": [C.c_char_p, C.c_char_p, P(SafetensorsInfo), SINK],
    "ullm_cuda_quantize_safetensors": [vp, C.c_char_p, C.c_char_p, P(Weight), SINK],
    "ullm_cuda_prepare": [vp, P(PlanOp), u32, P(vp), SINK],
    "ullm_cuda_prepared_destroy": [P(vp), SINK],
    "ullm_cuda_submit": [vp, vp, P(Binding), u32, P(vp), u32, P(vp), SINK],
    "ullm_cuda_event_query": [vp, P(u32), SINK],
    "ullm_cuda_event_wait": [vp, u32, SINK],
    "ullm_cuda_event_destroy": [P(vp), SINK],
    "ullm_cuda_context_shutdown": [vp, u32, P(u32), SINK],
    "ullm_cuda_linear_enqueue_partial": [vp, P(LinearDesc), P(Slots), SINK],
    "ullm_cuda_linear_enqueue_reduced": [vp, P(LinearDesc), P(Slots), Tensor, SINK],
    "ullm_cuda_comm_unique_id": [P(C.c_uint8), SINK],
    "ullm_cuda_comm_create": [vp, P(C.c_uint8), u32, u32, P(vp), SINK],
    "ullm_cuda_comm_all_reduce": [vp, vp, Tensor, u64, u32, SINK],
    "ullm_cuda_comm_destroy": [P(vp), SINK],
    "ullm_cuda_stack_create": [vp, vp, vp, P(StackDesc), P(vp), SINK],
    "ullm_cuda_stack_step": [vp, u64, Tensor, Tensor, SINK],
    "ullm_cuda_stack_step_host": [vp, u64, vp, vp, u32, SINK],
    "ullm_cuda_stack_linear_info": [vp, u32, u32, P(StackLinearInfo), SINK],
    "ullm_cuda_stack_stats": [vp, P(u64), P(u64), SINK],
    "ullm_cuda_stack_destroy": [P(vp), SINK],
}

_lib = None


def load():
    """Loads libullm_cuda.so and attaches the signatures.  Raises if the library
    or any declared symbol is missing: nothing here can run without it."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `make -C ullm-project_b200/csrc` "
                "(the CUDA library is the only implementation; there is no fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the export is missing
            fn.argtypes = argtypes
            fn.restype = u32
        _lib = lib
    return _lib

//! Raw declarations of the uLLM CUDA backend's C ABI (`include/ullm_cuda.h`, ABI version 1).
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain there); written by hand,
//! declaration by declaration, against the header.  `build.rs` compares every struct's size and the offsets of
//! its fields with a probe compiled from the header, which is what keeps this file honest.
//!
//! Counterpart of `crates/ullm-hip-sys/src/bindings.rs:100-119` (the four version / probe functions) extended by
//! the data plane the reference's HIP ABI does not have yet: contexts, queues, buffers, completions, the
//! quantisation routines, the quantised linear op, and the tensor-parallel stack.
#![allow(non_camel_case_types)]
#![allow(non_upper_case_globals)]

use core::ffi::{c_char, c_void};

pub type ullm_status_t = u32;

pub const ULLM_CUDA_ABI_VERSION: u32 = 1;
pub const ULLM_CUDA_LIBRARY_VERSION_MAJOR: u32 = 0;
pub const ULLM_CUDA_LIBRARY_VERSION_MINOR: u32 = 1;
pub const ULLM_CUDA_LIBRARY_VERSION_PATCH: u32 = 0;
pub const ULLM_STATUS_OK: ullm_status_t = 0;
pub const ULLM_STATUS_INVALID_ARGUMENT: ullm_status_t = 1;
pub const ULLM_STATUS_BUFFER_TOO_SMALL: ullm_status_t = 2;
pub const ULLM_STATUS_UNSUPPORTED: ullm_status_t = 3;
pub const ULLM_STATUS_INVALID_ABI_VERSION: ullm_status_t = 5;
pub const ULLM_STATUS_RESERVED_NONZERO: ullm_status_t = 6;
pub const ULLM_STATUS_INTERNAL_ERROR: ullm_status_t = 7;
pub const ULLM_STATUS_CUDA_UNAVAILABLE: ullm_status_t = 4;
pub const ULLM_STATUS_CUDA_TIMEOUT: ullm_status_t = 8;
pub const ULLM_STATUS_CUDA_INVALID_HANDLE: ullm_status_t = 9;
pub const ULLM_STATUS_CUDA_ZERO_DISPATCH: ullm_status_t = 10;
pub const ULLM_STATUS_CUDA_RUNTIME_ERROR: ullm_status_t = 11;
pub const ULLM_STATUS_CUDA_DISPATCH_CONTRACT: ullm_status_t = 12;
pub const ULLM_STATUS_CUDA_OUT_OF_MEMORY: ullm_status_t = 13;
pub const ULLM_STATUS_CUDA_OUT_OF_RANGE: ullm_status_t = 14;
pub const ULLM_STATUS_CUDA_COMM_ERROR: ullm_status_t = 15;
pub const ULLM_STATUS_CUDA_DEVICE_FLAGGED: ullm_status_t = 16;
pub const ULLM_BACKEND_CUDA: u32 = 2;
pub const ULLM_CUDA_DTYPE_BF16: u32 = 0;
pub const ULLM_CUDA_DTYPE_F16: u32 = 1;
pub const ULLM_CUDA_DTYPE_F32: u32 = 2;
pub const ULLM_CUDA_DTYPE_F8E4M3FN: u32 = 3;
pub const ULLM_CUDA_DTYPE_I8: u32 = 7;
pub const ULLM_CUDA_DTYPE_U8: u32 = 8;
pub const ULLM_CUDA_ENCODING_UNQUANTIZED: u32 = 0;
pub const ULLM_CUDA_ENCODING_NVFP4: u32 = 1;
pub const ULLM_CUDA_ENCODING_AQ4: u32 = 2;
pub const ULLM_CUDA_ENCODING_FP8_CHANNEL: u32 = 3;
pub const ULLM_CUDA_AQ4_GROUP: u32 = 128;
pub const ULLM_CUDA_PROLOGUE_NONE: u32 = 0;
pub const ULLM_CUDA_PROLOGUE_RMSNORM: u32 = 1;
pub const ULLM_CUDA_PROLOGUE_SWIGLU: u32 = 2;
pub const ULLM_CUDA_EPILOGUE_NONE: u32 = 0;
pub const ULLM_CUDA_EPILOGUE_SWIGLU: u32 = 1;
pub const ULLM_CUDA_KERNEL_AUTO: u32 = 0;
pub const ULLM_CUDA_KERNEL_MATVEC: u32 = 1;
pub const ULLM_CUDA_KERNEL_GEMM: u32 = 2;
pub const ULLM_CUDA_STACK_FLAG_NO_GRAPH: u32 = 1;
pub const ULLM_CUDA_STACK_FLAG_KEEP_ACTIVATIONS: u32 = 2;
pub const ULLM_CUDA_STACK_FLAG_NCCL_ONLY: u32 = 4;
pub const ULLM_CUDA_STACK_FLAG_GATHER_PER_BLOCK: u32 = 8;
pub const ULLM_CUDA_STACK_FLAG_GATHER_PER_CLUSTER: u32 = 16;
pub const ULLM_CUDA_STACK_LINEAR_QKV: u32 = 0;
pub const ULLM_CUDA_STACK_LINEAR_O: u32 = 1;
pub const ULLM_CUDA_STACK_LINEAR_GATE_UP: u32 = 2;
pub const ULLM_CUDA_STACK_LINEAR_DOWN: u32 = 3;
pub const ULLM_CUDA_STACK_LINEAR_LM_HEAD: u32 = 4;
pub const ULLM_CUDA_COMM_ID_BYTES: usize = 128;
pub const ULLM_CUDA_STATIC_SCRATCH_BYTES: u64 = 8 << 20;

#[repr(C)]
pub struct ullm_cuda_context_t {
    _private: [u8; 0],
}

#[repr(C)]
pub struct ullm_cuda_queue_t {
    _private: [u8; 0],
}

#[repr(C)]
pub struct ullm_cuda_buffer_t {
    _private: [u8; 0],
}

#[repr(C)]
pub struct ullm_cuda_completion_t {
    _private: [u8; 0],
}

#[repr(C)]
pub struct ullm_cuda_graph_t {
    _private: [u8; 0],
}

#[repr(C)]
pub struct ullm_cuda_comm_t {
    _private: [u8; 0],
}

#[repr(C)]
pub struct ullm_cuda_stack_t {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_error_sink_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub message: *mut c_char,
    pub message_capacity: u64,
    pub message_length: u64,
    pub reserved: [u64; 2],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_version_info_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub major: u32,
    pub minor: u32,
    pub patch: u32,
    pub reserved: [u32; 3],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_backend_probe_result_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub backend: u32,
    pub available: u32,
    pub cuda_runtime_present: u32,
    pub device_count: u32,
    pub sm_major: u32,
    pub sm_minor: u32,
    pub sm_count: u32,
    pub l2_bytes_mib: u32,
    pub global_memory_bytes: u64,
    pub reserved: [u32; 4],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_context_probe_result_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub context_present: u32,
    pub cuda_available: u32,
    pub device_ordinal: u32,
    pub reserved: [u32; 3],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_tensor_t {
    pub buffer: *mut ullm_cuda_buffer_t,
    pub offset_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_weight_t {
    pub encoding: u32,
    pub group_size: u32,
    pub n: u64,
    pub k: u64,
    pub values: ullm_cuda_tensor_t,
    pub scales: ullm_cuda_tensor_t,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_completion_result_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub dispatch_count: u64,
    pub copy_count: u64,
    pub selected_backend: u32,
    pub fallback_used: u32,
    pub terminal: u32,
    pub device_flags: u32,
    pub reserved: [u32; 4],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_linear_desc_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub weight: ullm_cuda_weight_t,
    pub m: u64,
    pub input: ullm_cuda_tensor_t,
    pub input_row_stride: u64,
    pub output: ullm_cuda_tensor_t,
    pub output_row_stride: u64,
    pub input_dtype: u32,
    pub output_dtype: u32,
    pub prologue: u32,
    pub kernel: u32,
    pub rms_eps: f32,
    pub epilogue: u32,
    pub norm_weight: ullm_cuda_tensor_t,
    pub residual: ullm_cuda_tensor_t,
    pub residual_row_stride: u64,
    pub reserved: [u32; 4],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_slots_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub slots: ullm_cuda_tensor_t,
    pub rank_stride_bytes: u64,
    pub ranks: u32,
    pub rank: u32,
    pub tag: u32,
    pub gather: u32,
    pub reserved: [u32; 4],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_stack_desc_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub encoding: u32,
    pub layers: u32,
    pub hidden: u32,
    pub q_heads: u32,
    pub kv_heads: u32,
    pub head_dim: u32,
    pub ffn: u32,
    pub vocab: u32,
    pub tp_rank: u32,
    pub tp_size: u32,
    pub max_tokens: u32,
    pub flags: u32,
    pub seed: u64,
    pub rms_eps: f32,
    pub reserved: [u32; 5],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ullm_cuda_stack_linear_info_t {
    pub struct_size: u32,
    pub abi_version: u32,
    pub weight: ullm_cuda_weight_t,
    pub tensor_id: u64,
    pub full_n: u64,
    pub full_k: u64,
    pub row_begin: u64,
    pub col_begin: u64,
    pub last_input: ullm_cuda_tensor_t,
    pub last_output: ullm_cuda_tensor_t,
    pub input_dtype: u32,
    pub output_dtype: u32,
    pub prologue: u32,
    pub epilogue: u32,
    pub norm_weight: ullm_cuda_tensor_t,
    pub last_residual: ullm_cuda_tensor_t,
    pub norm_tensor_id: u64,
    pub reserved: [u32; 4],
}

unsafe extern "C" {
    pub fn ullm_cuda_get_abi_version(
        abi_version: *mut u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_query_version(
        version: *mut ullm_cuda_version_info_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_backend_probe(
        backend: u32,
        result: *mut ullm_cuda_backend_probe_result_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_context_probe(
        context: *const ullm_cuda_context_t,
        result: *mut ullm_cuda_context_probe_result_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_context_create(
        device_ordinal: u32,
        context: *mut *mut ullm_cuda_context_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_context_destroy(
        context: *mut *mut ullm_cuda_context_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_context_set_wait_limit(
        context: *mut ullm_cuda_context_t,
        limit_ms: u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_queue_create(
        context: *mut ullm_cuda_context_t,
        queue: *mut *mut ullm_cuda_queue_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_queue_destroy(
        queue: *mut *mut ullm_cuda_queue_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_buffer_alloc(
        context: *mut ullm_cuda_context_t,
        size_bytes: u64,
        buffer: *mut *mut ullm_cuda_buffer_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_buffer_free(
        buffer: *mut *mut ullm_cuda_buffer_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_buffer_size(
        buffer: *const ullm_cuda_buffer_t,
        size_bytes: *mut u64,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_buffer_upload(
        queue: *mut ullm_cuda_queue_t,
        dst: ullm_cuda_tensor_t,
        host_src: *const c_void,
        size_bytes: u64,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_buffer_download(
        queue: *mut ullm_cuda_queue_t,
        src: ullm_cuda_tensor_t,
        host_dst: *mut c_void,
        size_bytes: u64,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_buffer_fill(
        queue: *mut ullm_cuda_queue_t,
        dst: ullm_cuda_tensor_t,
        value: u8,
        size_bytes: u64,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_queue_signal(
        queue: *mut ullm_cuda_queue_t,
        completion: *mut *mut ullm_cuda_completion_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_completion_wait(
        completion: *mut ullm_cuda_completion_t,
        timeout_ms: u32,
        result: *mut ullm_cuda_completion_result_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_completion_elapsed_ms(
        start: *mut ullm_cuda_completion_t,
        end: *mut ullm_cuda_completion_t,
        milliseconds: *mut f32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_completion_query(
        completion: *mut ullm_cuda_completion_t,
        timeout_ms: u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_completion_destroy(
        completion: *mut *mut ullm_cuda_completion_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_queue_capture_begin(
        queue: *mut ullm_cuda_queue_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_queue_capture_end(
        queue: *mut ullm_cuda_queue_t,
        graph: *mut *mut ullm_cuda_graph_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_graph_launch(
        graph: *mut ullm_cuda_graph_t,
        queue: *mut ullm_cuda_queue_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_graph_destroy(
        graph: *mut *mut ullm_cuda_graph_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_synth_weights(
        queue: *mut ullm_cuda_queue_t,
        seed: u64,
        tensor_id: u64,
        first_element: u64,
        count: u64,
        std: f32,
        out_f32: ullm_cuda_tensor_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_synth_activations(
        queue: *mut ullm_cuda_queue_t,
        seed: u64,
        tensor_id: u64,
        first_element: u64,
        count: u64,
        out_bf16: ullm_cuda_tensor_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_quantize(
        queue: *mut ullm_cuda_queue_t,
        src_f32: ullm_cuda_tensor_t,
        weight: *const ullm_cuda_weight_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_aq4_unpack(
        queue: *mut ullm_cuda_queue_t,
        weight: *const ullm_cuda_weight_t,
        out_i8: ullm_cuda_tensor_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_aq4_pack(
        queue: *mut ullm_cuda_queue_t,
        src_i8: ullm_cuda_tensor_t,
        weight: *const ullm_cuda_weight_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_dequantize(
        queue: *mut ullm_cuda_queue_t,
        weight: *const ullm_cuda_weight_t,
        out: ullm_cuda_tensor_t,
        out_dtype: u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_linear_supports(
        desc: *const ullm_cuda_linear_desc_t,
        selected_kernel: *mut u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_linear_enqueue(
        queue: *mut ullm_cuda_queue_t,
        desc: *const ullm_cuda_linear_desc_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_linear_submit(
        queue: *mut ullm_cuda_queue_t,
        desc: *const ullm_cuda_linear_desc_t,
        completion: *mut *mut ullm_cuda_completion_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_linear_enqueue_static_scratch(
        queue: *mut ullm_cuda_queue_t,
        desc: *const ullm_cuda_linear_desc_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_linear_enqueue_partial(
        queue: *mut ullm_cuda_queue_t,
        desc: *const ullm_cuda_linear_desc_t,
        slots: *const ullm_cuda_slots_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_linear_enqueue_reduced(
        queue: *mut ullm_cuda_queue_t,
        desc: *const ullm_cuda_linear_desc_t,
        slots: *const ullm_cuda_slots_t,
        reduced_out: ullm_cuda_tensor_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_comm_unique_id(
        id: *mut u8,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_comm_create(
        context: *mut ullm_cuda_context_t,
        id: *const u8,
        rank: u32,
        size: u32,
        comm: *mut *mut ullm_cuda_comm_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_comm_all_reduce(
        comm: *mut ullm_cuda_comm_t,
        queue: *mut ullm_cuda_queue_t,
        data: ullm_cuda_tensor_t,
        count: u64,
        dtype: u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_comm_destroy(
        comm: *mut *mut ullm_cuda_comm_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_stack_create(
        context: *mut ullm_cuda_context_t,
        queue: *mut ullm_cuda_queue_t,
        comm: *mut ullm_cuda_comm_t,
        desc: *const ullm_cuda_stack_desc_t,
        stack: *mut *mut ullm_cuda_stack_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_stack_step(
        stack: *mut ullm_cuda_stack_t,
        m: u64,
        input_bf16: ullm_cuda_tensor_t,
        output_bf16: ullm_cuda_tensor_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_stack_step_host(
        stack: *mut ullm_cuda_stack_t,
        m: u64,
        host_input_bf16: *const c_void,
        host_output_bf16: *mut c_void,
        timeout_ms: u32,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_stack_linear_info(
        stack: *mut ullm_cuda_stack_t,
        layer: u32,
        which: u32,
        info: *mut ullm_cuda_stack_linear_info_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_stack_stats(
        stack: *mut ullm_cuda_stack_t,
        weight_bytes: *mut u64,
        launches_per_step: *mut u64,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
    pub fn ullm_cuda_stack_destroy(
        stack: *mut *mut ullm_cuda_stack_t,
        error_sink: *mut ullm_cuda_error_sink_t,
    ) -> ullm_status_t;
}

/// Metadata of this hand-written mirror (the reference records the same for its bindgen output,
/// `crates/ullm-hip-sys/src/lib.rs:15-21`).
pub mod binding_metadata {
    pub const SOURCE: &str = "include/ullm_cuda.h";
    pub const ABI_VERSION: u32 = 1;
    pub const TOOL: &str = "hand-written; layouts verified by build.rs against a probe compiled from the header";
}

//! Safe wrapper of the CUDA (sm_100a) backend's C ABI.
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain there).  It follows
//! `ullm-cuda-sys` declaration by declaration; the same calls, in the same order, are exercised on a GPU by the
//! C++17 mirror `include/ullm_cuda.hpp` and by the Python mirror the parity tests use.
//!
//! Shaped after the reference's safe HIP wrapper, item by item:
//!   * `Status` with `from_raw` / `raw`                       crates/ullm-hip/src/lib.rs:20-76
//!   * an error type carrying status + native diagnostic       crates/ullm-hip/src/lib.rs:78-110
//!   * caller-owned error sink of `ERROR_CAPACITY` bytes       crates/ullm-hip/src/lib.rs:154-187
//!   * `abi_version()`, `version()`, `backend_probe()`         crates/ullm-hip/src/lib.rs:189-268
//!   * submit -> `wait(self, timeout)` consumes the completion crates/ullm-hip/src/lib.rs:293-441
//!   * `connect()` only after an available probe; `Backend`    crates/ullm-hip/src/lib.rs:470-513
//! Unlike the reference's Phase-1 wrapper this backend executes numerical work — on the GPU only.  A missing
//! library or device is an error (`Status::CudaUnavailable`), never a fallback to the CPU.
#![forbid(unsafe_op_in_unsafe_fn)]

use std::fmt;
use std::mem::size_of;
use std::ptr::{self, NonNull};
use std::sync::Arc;
use std::time::Duration;

use ullm_core::{
    AccessMode, Backend, BackendCapabilities, BackendError, BackendSupport, BufferHandle, BufferUse,
    CompletionLease, DType, Encoding, EventHandle, ExecutionReceipt, MaterializedTensor, QueueHandle,
    SemanticOp, SemanticOpKind, TensorView,
};
use ullm_cuda_sys as sys;

const ERROR_CAPACITY: usize = 512;

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum Status {
    Ok,
    InvalidArgument,
    BufferTooSmall,
    Unsupported,
    CudaUnavailable,
    InvalidAbiVersion,
    ReservedNonzero,
    InternalError,
    Timeout,
    InvalidHandle,
    ZeroDispatch,
    RuntimeError,
    DispatchContract,
    OutOfMemory,
    OutOfRange,
    CommError,
    DeviceFlagged,
    Unknown(u32),
}

impl Status {
    pub const fn from_raw(raw: u32) -> Self {
        match raw {
            sys::ULLM_STATUS_OK => Self::Ok,
            sys::ULLM_STATUS_INVALID_ARGUMENT => Self::InvalidArgument,
            sys::ULLM_STATUS_BUFFER_TOO_SMALL => Self::BufferTooSmall,
            sys::ULLM_STATUS_UNSUPPORTED => Self::Unsupported,
            sys::ULLM_STATUS_CUDA_UNAVAILABLE => Self::CudaUnavailable,
            sys::ULLM_STATUS_INVALID_ABI_VERSION => Self::InvalidAbiVersion,
            sys::ULLM_STATUS_RESERVED_NONZERO => Self::ReservedNonzero,
            sys::ULLM_STATUS_INTERNAL_ERROR => Self::InternalError,
            sys::ULLM_STATUS_CUDA_TIMEOUT => Self::Timeout,
            sys::ULLM_STATUS_CUDA_INVALID_HANDLE => Self::InvalidHandle,
            sys::ULLM_STATUS_CUDA_ZERO_DISPATCH => Self::ZeroDispatch,
            sys::ULLM_STATUS_CUDA_RUNTIME_ERROR => Self::RuntimeError,
            sys::ULLM_STATUS_CUDA_DISPATCH_CONTRACT => Self::DispatchContract,
            sys::ULLM_STATUS_CUDA_OUT_OF_MEMORY => Self::OutOfMemory,
            sys::ULLM_STATUS_CUDA_OUT_OF_RANGE => Self::OutOfRange,
            sys::ULLM_STATUS_CUDA_COMM_ERROR => Self::CommError,
            sys::ULLM_STATUS_CUDA_DEVICE_FLAGGED => Self::DeviceFlagged,
            other => Self::Unknown(other),
        }
    }

    pub const fn raw(self) -> u32 {
        match self {
            Self::Ok => sys::ULLM_STATUS_OK,
            Self::InvalidArgument => sys::ULLM_STATUS_INVALID_ARGUMENT,
            Self::BufferTooSmall => sys::ULLM_STATUS_BUFFER_TOO_SMALL,
            Self::Unsupported => sys::ULLM_STATUS_UNSUPPORTED,
            Self::CudaUnavailable => sys::ULLM_STATUS_CUDA_UNAVAILABLE,
            Self::InvalidAbiVersion => sys::ULLM_STATUS_INVALID_ABI_VERSION,
            Self::ReservedNonzero => sys::ULLM_STATUS_RESERVED_NONZERO,
            Self::InternalError => sys::ULLM_STATUS_INTERNAL_ERROR,
            Self::Timeout => sys::ULLM_STATUS_CUDA_TIMEOUT,
            Self::InvalidHandle => sys::ULLM_STATUS_CUDA_INVALID_HANDLE,
            Self::ZeroDispatch => sys::ULLM_STATUS_CUDA_ZERO_DISPATCH,
            Self::RuntimeError => sys::ULLM_STATUS_CUDA_RUNTIME_ERROR,
            Self::DispatchContract => sys::ULLM_STATUS_CUDA_DISPATCH_CONTRACT,
            Self::OutOfMemory => sys::ULLM_STATUS_CUDA_OUT_OF_MEMORY,
            Self::OutOfRange => sys::ULLM_STATUS_CUDA_OUT_OF_RANGE,
            Self::CommError => sys::ULLM_STATUS_CUDA_COMM_ERROR,
            Self::DeviceFlagged => sys::ULLM_STATUS_CUDA_DEVICE_FLAGGED,
            Self::Unknown(raw) => raw,
        }
    }
}

/// A non-OK status of the native library with its diagnostic text.
#[derive(Clone, Debug, Eq, PartialEq)]
pub struct CudaError {
    pub status: Status,
    pub message: String,
}

impl fmt::Display for CudaError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "{:?}: {}", self.status, self.message)
    }
}

impl std::error::Error for CudaError {}

pub type Result<T> = std::result::Result<T, CudaError>;

/// One native call with a fresh caller-owned error sink (the callee keeps no pointer to it).
fn call(f: impl FnOnce(*mut sys::ullm_cuda_error_sink_t) -> u32) -> Result<()> {
    let mut buffer = [0u8; ERROR_CAPACITY];
    let mut sink = sys::ullm_cuda_error_sink_t {
        struct_size: size_of::<sys::ullm_cuda_error_sink_t>() as u32,
        abi_version: sys::ULLM_CUDA_ABI_VERSION,
        message: buffer.as_mut_ptr().cast(),
        message_capacity: buffer.len() as u64,
        message_length: 0,
        reserved: [0, 0],
    };
    let raw = f(&mut sink);
    if raw == sys::ULLM_STATUS_OK {
        return Ok(());
    }
    let len = usize::try_from(sink.message_length).unwrap_or(buffer.len()).min(buffer.len() - 1);
    Err(CudaError { status: Status::from_raw(raw), message: String::from_utf8_lossy(&buffer[..len]).into_owned() })
}

pub fn abi_version() -> Result<u32> {
    let mut v = 0u32;
    call(|s| unsafe { sys::ullm_cuda_get_abi_version(&mut v, s) })?;
    Ok(v)
}

#[derive(Clone, Debug, Eq, PartialEq)]
pub struct BackendProbe {
    pub available: bool,
    pub cuda_runtime_present: bool,
    pub device_count: u32,
    pub sm: (u32, u32),
    pub sm_count: u32,
    pub global_memory_bytes: u64,
    pub diagnostic: String,
}

/// `CudaUnavailable` is a result of the probe, not a failure (crates/ullm-hip/src/lib.rs:230-242).
pub fn backend_probe() -> Result<BackendProbe> {
    let mut r: sys::ullm_cuda_backend_probe_result_t = unsafe { std::mem::zeroed() };
    r.struct_size = size_of::<sys::ullm_cuda_backend_probe_result_t>() as u32;
    r.abi_version = sys::ULLM_CUDA_ABI_VERSION;
    let outcome = call(|s| unsafe { sys::ullm_cuda_backend_probe(sys::ULLM_BACKEND_CUDA, &mut r, s) });
    let diagnostic = match outcome {
        Ok(()) => String::new(),
        Err(e) if e.status == Status::CudaUnavailable => e.message,
        Err(e) => return Err(e),
    };
    Ok(BackendProbe {
        available: r.available != 0,
        cuda_runtime_present: r.cuda_runtime_present != 0,
        device_count: r.device_count,
        sm: (r.sm_major, r.sm_minor),
        sm_count: r.sm_count,
        global_memory_bytes: r.global_memory_bytes,
        diagnostic,
    })
}

macro_rules! owned_handle {
    ($name:ident, $raw:ty, $destroy:path) => {
        pub struct $name {
            raw: NonNull<$raw>,
        }
        // The native objects are guarded by their own mutexes (Backend: Send + Sync, backend.rs:5).
        unsafe impl Send for $name {}
        unsafe impl Sync for $name {}
        impl $name {
            fn as_ptr(&self) -> *mut $raw {
                self.raw.as_ptr()
            }
        }
        impl Drop for $name {
            fn drop(&mut self) {
                // never blocks: the library retires what may still be in use once its completion is proven
                let mut p = self.raw.as_ptr();
                let _ = call(|s| unsafe { $destroy(&mut p, s) });
            }
        }
    };
}

owned_handle!(Context, sys::ullm_cuda_context_t, sys::ullm_cuda_context_destroy);
owned_handle!(Queue, sys::ullm_cuda_queue_t, sys::ullm_cuda_queue_destroy);
owned_handle!(Buffer, sys::ullm_cuda_buffer_t, sys::ullm_cuda_buffer_free);

fn non_null<T>(p: *mut T, what: &str) -> Result<NonNull<T>> {
    NonNull::new(p).ok_or_else(|| CudaError { status: Status::InternalError, message: format!("native {what} returned null") })
}

impl Context {
    pub fn create(device_ordinal: u32) -> Result<Arc<Self>> {
        let mut p = ptr::null_mut();
        call(|s| unsafe { sys::ullm_cuda_context_create(device_ordinal, &mut p, s) })?;
        Ok(Arc::new(Self { raw: non_null(p, "context create")? }))
    }

    /// Limit of every device-side wait of kernels launched for this context from now on.
    pub fn set_wait_limit(&self, limit: Duration) -> Result<()> {
        let ms = limit.as_millis().try_into().unwrap_or(u32::MAX);
        call(|s| unsafe { sys::ullm_cuda_context_set_wait_limit(self.as_ptr(), ms, s) })
    }
}

impl Queue {
    pub fn create(ctx: &Context) -> Result<Self> {
        let mut p = ptr::null_mut();
        call(|s| unsafe { sys::ullm_cuda_queue_create(ctx.as_ptr(), &mut p, s) })?;
        Ok(Self { raw: non_null(p, "queue create")? })
    }

    /// Copies during the call: the library keeps no pointer to `data` after returning
    /// (docs/architecture/runtime.md:47, :77 of the reference).
    pub fn upload(&self, dst: Span<'_>, data: &[u8]) -> Result<()> {
        call(|s| unsafe { sys::ullm_cuda_buffer_upload(self.as_ptr(), dst.raw(), data.as_ptr().cast(), data.len() as u64, s) })
    }

    pub fn download(&self, src: Span<'_>, out: &mut [u8]) -> Result<()> {
        call(|s| unsafe { sys::ullm_cuda_buffer_download(self.as_ptr(), src.raw(), out.as_mut_ptr().cast(), out.len() as u64, s) })
    }

    pub fn signal(&self) -> Result<Completion> {
        let mut p = ptr::null_mut();
        call(|s| unsafe { sys::ullm_cuda_queue_signal(self.as_ptr(), &mut p, s) })?;
        Ok(Completion { raw: Some(non_null(p, "queue signal")?) })
    }
}

impl Buffer {
    pub fn alloc(ctx: &Context, bytes: u64) -> Result<Arc<Self>> {
        let mut p = ptr::null_mut();
        call(|s| unsafe { sys::ullm_cuda_buffer_alloc(ctx.as_ptr(), bytes, &mut p, s) })?;
        Ok(Arc::new(Self { raw: non_null(p, "buffer alloc")? }))
    }

    pub fn at(&self, offset_bytes: u64) -> Span<'_> {
        Span { buffer: self, offset_bytes }
    }
}

/// A span inside a device buffer; every op bounds-checks it on the host before launching anything.
#[derive(Clone, Copy)]
pub struct Span<'a> {
    buffer: &'a Buffer,
    offset_bytes: u64,
}

impl Span<'_> {
    fn raw(self) -> sys::ullm_cuda_tensor_t {
        sys::ullm_cuda_tensor_t { buffer: self.buffer.as_ptr(), offset_bytes: self.offset_bytes }
    }
}

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct CompletionReport {
    pub dispatch_count: u64,
    pub copy_count: u64,
    pub selected_backend: u32,
    pub fallback_used: bool,
    pub device_flags: u32,
}

/// submit -> wait -> drop.  `wait` takes `self`: the native handle is consumed by every outcome, a timeout
/// included (native/hip/src/hip_evidence_runtime.hip.cpp:691-716 sets the same rule).
pub struct Completion {
    raw: Option<NonNull<sys::ullm_cuda_completion_t>>,
}

impl Completion {
    pub fn wait(mut self, timeout: Duration) -> Result<CompletionReport> {
        let handle = self.raw.take().expect("a completion is waited on once");
        let mut r: sys::ullm_cuda_completion_result_t = unsafe { std::mem::zeroed() };
        r.struct_size = size_of::<sys::ullm_cuda_completion_result_t>() as u32;
        r.abi_version = sys::ULLM_CUDA_ABI_VERSION;
        let ms = timeout.as_millis().try_into().unwrap_or(u32::MAX); // saturates like lib.rs:400-402
        call(|s| unsafe { sys::ullm_cuda_completion_wait(handle.as_ptr(), ms, &mut r, s) })?;
        let report = CompletionReport {
            dispatch_count: r.dispatch_count,
            copy_count: r.copy_count,
            selected_backend: r.selected_backend,
            fallback_used: r.fallback_used != 0,
            device_flags: r.device_flags,
        };
        // the same contract the reference re-checks on every run (crates/ullm-hip/src/lib.rs:404-430)
        if report.selected_backend != sys::ULLM_BACKEND_CUDA || report.fallback_used {
            return Err(CudaError { status: Status::DispatchContract, message: "completion reports a fallback".to_owned() });
        }
        Ok(report)
    }

    /// Single poll that keeps the completion.
    pub fn reached(&self) -> Result<bool> {
        let handle = self.raw.expect("completion not yet waited on");
        match call(|s| unsafe { sys::ullm_cuda_completion_query(handle.as_ptr(), 0, s) }) {
            Ok(()) => Ok(true),
            Err(e) if e.status == Status::Timeout => Ok(false),
            Err(e) => Err(e),
        }
    }
}

impl Drop for Completion {
    fn drop(&mut self) {
        if let Some(h) = self.raw.take() {
            let mut p = h.as_ptr();
            let _ = call(|s| unsafe { sys::ullm_cuda_completion_destroy(&mut p, s) });
        }
    }
}

/// The additive quantised encodings (see ullm-core-additions.md) as this backend names them.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum WeightEncoding {
    /// 4-bit symmetric codes, two per byte, one f16 scale per group of 128 along K.
    Aq4,
    /// e4m3fn codes, one f32 scale per output channel.
    Fp8Channel,
}

/// y[M,N] = prologue(x)[M,K] . W'[N,K]^T (+ residual), fp32 accumulate: the op `SemanticOpKind::QuantLinear` names.
pub struct QuantLinear<'a> {
    pub encoding: WeightEncoding,
    pub m: u64,
    pub n: u64,
    pub k: u64,
    pub weight_values: Span<'a>,
    pub weight_scales: Span<'a>,
    pub input: Span<'a>,
    pub output: Span<'a>,
    pub input_dtype: DType,
    pub output_dtype: DType,
    pub rmsnorm: Option<(f32, Option<Span<'a>>)>, // (eps, gamma)
    pub residual: Option<Span<'a>>,
}

fn dtype_id(d: DType) -> u32 {
    match d {
        DType::Bf16 => sys::ULLM_CUDA_DTYPE_BF16,
        DType::F16 => sys::ULLM_CUDA_DTYPE_F16,
        DType::F32 => sys::ULLM_CUDA_DTYPE_F32,
        DType::F8E4M3Fn => sys::ULLM_CUDA_DTYPE_F8E4M3FN,
        DType::U8 => sys::ULLM_CUDA_DTYPE_U8,
        _ => u32::MAX, // rejected by the native validation as UNSUPPORTED
    }
}

impl QuantLinear<'_> {
    fn desc(&self) -> sys::ullm_cuda_linear_desc_t {
        let mut d: sys::ullm_cuda_linear_desc_t = unsafe { std::mem::zeroed() };
        d.struct_size = size_of::<sys::ullm_cuda_linear_desc_t>() as u32;
        d.abi_version = sys::ULLM_CUDA_ABI_VERSION;
        d.weight.encoding = match self.encoding {
            WeightEncoding::Aq4 => sys::ULLM_CUDA_ENCODING_AQ4,
            WeightEncoding::Fp8Channel => sys::ULLM_CUDA_ENCODING_FP8_CHANNEL,
        };
        d.weight.group_size = if self.encoding == WeightEncoding::Aq4 { sys::ULLM_CUDA_AQ4_GROUP } else { 0 };
        d.weight.n = self.n;
        d.weight.k = self.k;
        d.weight.values = self.weight_values.raw();
        d.weight.scales = self.weight_scales.raw();
        d.m = self.m;
        d.input = self.input.raw();
        d.output = self.output.raw();
        d.input_dtype = dtype_id(self.input_dtype);
        d.output_dtype = dtype_id(self.output_dtype);
        if let Some((eps, gamma)) = self.rmsnorm {
            d.prologue = sys::ULLM_CUDA_PROLOGUE_RMSNORM;
            d.rms_eps = eps;
            if let Some(g) = gamma {
                d.norm_weight = g.raw();
            }
        }
        if let Some(r) = self.residual {
            d.residual = r.raw();
        }
        d
    }
}

impl Queue {
    /// Quantises f32 values already on the device into the weight this op describes (its `weight_values` /
    /// `weight_scales` spans); bytes are identical to the format specification's.
    pub fn quantize(&self, src_f32: Span<'_>, op: &QuantLinear<'_>) -> Result<()> {
        let d = op.desc();
        call(|s| unsafe { sys::ullm_cuda_quantize(self.as_ptr(), src_f32.raw(), &d.weight, s) })
    }

    /// Load-time path: reads the named tensor of a safetensors file (F32 / F16 / BF16) chunk by chunk and
    /// quantises it on the device into the op's weight spans.
    pub fn quantize_safetensors(&self, path: &std::ffi::CStr, tensor_name: &std::ffi::CStr, op: &QuantLinear<'_>) -> Result<()> {
        let d = op.desc();
        call(|s| unsafe { sys::ullm_cuda_quantize_safetensors(self.as_ptr(), path.as_ptr(), tensor_name.as_ptr(), &d.weight, s) })
    }
}

// ---- coarse command lists (docs/architecture/runtime.md:53-63, :77-79 of the reference) -------------------------

owned_handle!(Prepared, sys::ullm_cuda_prepared_t, sys::ullm_cuda_prepared_destroy);
owned_handle!(Event, sys::ullm_cuda_event_t, sys::ullm_cuda_event_destroy);

/// Which tensor of an op a binding supplies.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum Slot {
    WeightValues,
    WeightScales,
    Input,
    Output,
    NormWeight,
    Residual,
}

/// One (op, slot) -> span binding with the access the submission is allowed (ullm-core handles.rs:12-16).
pub struct Binding<'a> {
    pub op_index: u32,
    pub slot: Slot,
    pub access: AccessMode,
    pub span: Span<'a>,
}

/// Terminal state of a submission as its event reports it.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum EventState {
    Pending,
    Success,
    Failure,
}

impl Prepared {
    /// Shape-only descriptions of the ops (no spans): metadata is copied and kernels are chosen here, so
    /// `UNSUPPORTED` shows at prepare time, never at submit.
    pub fn new(ctx: &Context, ops: &[QuantLinear<'_>]) -> Result<Self> {
        let raw_ops: Vec<sys::ullm_cuda_plan_op_t> = ops
            .iter()
            .map(|op| {
                let d = op.desc();
                let mut o: sys::ullm_cuda_plan_op_t = unsafe { std::mem::zeroed() };
                o.struct_size = size_of::<sys::ullm_cuda_plan_op_t>() as u32;
                o.abi_version = sys::ULLM_CUDA_ABI_VERSION;
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
                if matches!(op.rmsnorm, Some((_, Some(_)))) {
                    o.flags |= sys::ULLM_CUDA_PLAN_OP_HAS_NORM_WEIGHT;
                }
                if op.residual.is_some() {
                    o.flags |= sys::ULLM_CUDA_PLAN_OP_HAS_RESIDUAL;
                }
                o
            })
            .collect();
        let mut p = ptr::null_mut();
        call(|s| unsafe { sys::ullm_cuda_prepare(ctx.as_ptr(), raw_ops.as_ptr(), raw_ops.len() as u32, &mut p, s) })?;
        Ok(Self { raw: non_null(p, "prepare")? })
    }

    /// Enqueues the prepared ops on `queue` behind `wait_for`; the bindings are checked against what each op reads
    /// and writes before anything is launched.  The returned event never blocks when dropped: the executor keeps
    /// watching the submission.
    pub fn submit(&self, queue: &Queue, bindings: &[Binding<'_>], wait_for: &[&Event]) -> Result<Event> {
        let raw_bindings: Vec<sys::ullm_cuda_binding_t> = bindings
            .iter()
            .map(|b| {
                let mut r: sys::ullm_cuda_binding_t = unsafe { std::mem::zeroed() };
                r.struct_size = size_of::<sys::ullm_cuda_binding_t>() as u32;
                r.abi_version = sys::ULLM_CUDA_ABI_VERSION;
                r.op_index = b.op_index;
                r.slot = match b.slot {
                    Slot::WeightValues => sys::ULLM_CUDA_SLOT_WEIGHT_VALUES,
                    Slot::WeightScales => sys::ULLM_CUDA_SLOT_WEIGHT_SCALES,
                    Slot::Input => sys::ULLM_CUDA_SLOT_INPUT,
                    Slot::Output => sys::ULLM_CUDA_SLOT_OUTPUT,
                    Slot::NormWeight => sys::ULLM_CUDA_SLOT_NORM_WEIGHT,
                    Slot::Residual => sys::ULLM_CUDA_SLOT_RESIDUAL,
                };
                r.access = match b.access {
                    AccessMode::Read => sys::ULLM_CUDA_ACCESS_READ,
                    AccessMode::Write => sys::ULLM_CUDA_ACCESS_WRITE,
                    AccessMode::ReadWrite => sys::ULLM_CUDA_ACCESS_READ_WRITE,
                };
                r.tensor = b.span.raw();
                r
            })
            .collect();
        let waits: Vec<*mut sys::ullm_cuda_event_t> = wait_for.iter().map(|e| e.as_ptr()).collect();
        let mut ev = ptr::null_mut();
        call(|s| unsafe {
            sys::ullm_cuda_submit(
                queue.as_ptr(),
                self.as_ptr(),
                raw_bindings.as_ptr(),
                raw_bindings.len() as u32,
                if waits.is_empty() { ptr::null() } else { waits.as_ptr() },
                waits.len() as u32,
                &mut ev,
                s,
            )
        })?;
        Ok(Event { raw: non_null(ev, "submit")? })
    }
}

impl Event {
    /// One poll; never consumes the event.  A failure after enqueue is this event's stored status.
    pub fn query(&self) -> Result<EventState> {
        let mut state = sys::ULLM_CUDA_EVENT_PENDING;
        call(|s| unsafe { sys::ullm_cuda_event_query(self.as_ptr(), &mut state, s) })?;
        Ok(match state {
            sys::ULLM_CUDA_EVENT_SUCCESS => EventState::Success,
            sys::ULLM_CUDA_EVENT_FAILURE => EventState::Failure,
            _ => EventState::Pending,
        })
    }

    /// Polls until the submission is terminal or the timeout runs out (`Status::Timeout`); the event stays usable.
    pub fn wait(&self, timeout: Duration) -> Result<()> {
        let ms = timeout.as_millis().try_into().unwrap_or(u32::MAX);
        call(|s| unsafe { sys::ullm_cuda_event_wait(self.as_ptr(), ms, s) })
    }
}

impl Context {
    /// Refuses new submissions, drains those in flight for at most `timeout`, and returns how many ended in failure
    /// (the executor's shutdown of docs/architecture/runtime.md:61-63).
    pub fn shutdown(&self, timeout: Duration) -> Result<u32> {
        let ms = timeout.as_millis().try_into().unwrap_or(u32::MAX);
        let mut failed = 0u32;
        call(|s| unsafe { sys::ullm_cuda_context_shutdown(self.as_ptr(), ms, &mut failed, s) })?;
        Ok(failed)
    }
}

/// Which kernel `supports` selected: the CUDA-core streaming matvec or the tcgen05 GEMM.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum Kernel {
    Matvec,
    Gemm,
}

/// A typed backend handle is only constructible after an available probe (crates/ullm-hip/src/lib.rs:470-485).
pub struct CudaBackend {
    context: Arc<Context>,
}

impl CudaBackend {
    pub fn connect(device_ordinal: u32) -> Result<Self> {
        let probe = backend_probe()?;
        if !probe.available {
            return Err(CudaError { status: Status::CudaUnavailable, message: probe.diagnostic });
        }
        Ok(Self { context: Context::create(device_ordinal)? })
    }

    pub fn context(&self) -> &Arc<Context> {
        &self.context
    }

    /// Shape-only answer: neither handles nor the device are consulted.
    pub fn supports_linear(op: &QuantLinear<'_>) -> Result<Kernel> {
        let d = op.desc();
        let mut k = 0u32;
        call(|s| unsafe { sys::ullm_cuda_linear_supports(&d, &mut k, s) })?;
        Ok(if k == sys::ULLM_CUDA_KERNEL_GEMM { Kernel::Gemm } else { Kernel::Matvec })
    }

    /// Buffer-binding execution as an inherent method: `Backend::execute` has no data plane
    /// (crates/ullm-core/src/backend.rs:5-11).  Returns the completion to wait on together with the
    /// ownership-only lease of `ullm-core` (crates/ullm-core/src/handles.rs:100-145) that keeps queue, event
    /// and buffers alive, with their access modes, until a higher layer has observed completion.
    pub fn submit_linear(&self, queue: &Queue, op: &QuantLinear<'_>, ids: LeaseIds) -> Result<(Completion, CompletionLease)> {
        let d = op.desc();
        let mut p = ptr::null_mut();
        call(|s| unsafe { sys::ullm_cuda_linear_submit(queue.as_ptr(), &d, &mut p, s) })?;
        let completion = Completion { raw: Some(non_null(p, "linear submit")?) };
        let mut uses = vec![
            BufferUse::new(ids.weights.clone(), AccessMode::Read),
            BufferUse::new(ids.input.clone(), AccessMode::Read),
            BufferUse::new(ids.output.clone(), if op.residual.is_some() { AccessMode::ReadWrite } else { AccessMode::Write }),
        ];
        uses.dedup_by(|a, b| a.buffer() == b.buffer());
        Ok((completion, CompletionLease::new(ids.queue, ids.event, uses)))
    }
}

/// Backend-independent identities of the objects one submission uses (the core never dereferences them).
pub struct LeaseIds {
    pub queue: Arc<QueueHandle>,
    pub event: Arc<EventHandle>,
    pub weights: Arc<BufferHandle>,
    pub input: Arc<BufferHandle>,
    pub output: Arc<BufferHandle>,
}

impl Backend for CudaBackend {
    fn name(&self) -> &'static str {
        "cuda"
    }

    fn capabilities(&self) -> BackendCapabilities {
        BackendCapabilities { metadata_only: false, numerical_execution: true, max_materialization_bytes: None }
    }

    /// Answers from kind, shapes and encodings alone, like the native `ullm_cuda_linear_supports`.
    fn supports(&self, operation: &SemanticOp) -> BackendSupport {
        match operation.kind() {
            SemanticOpKind::QuantLinear => match operation.operands() {
                [x, w, y] => {
                    let enc_ok = matches!(w.encoding(), Encoding::Aq4 { group_size: 128, scale_dtype: DType::F16 } | Encoding::Fp8Channel);
                    let k = w.shape().get(1).copied().unwrap_or(0);
                    let k_ok = match w.encoding() {
                        Encoding::Aq4 { .. } => k % 128 == 0,
                        _ => k % 16 == 0,
                    };
                    if enc_ok && k_ok && matches!(x.dtype(), DType::Bf16 | DType::F32) && matches!(y.dtype(), DType::Bf16 | DType::F32) {
                        BackendSupport::Supported
                    } else {
                        BackendSupport::Unsupported { reason: "quantised linear: AQ4 (group 128, f16 scales, K % 128 == 0) or FP8 per-channel (K % 16 == 0), bf16 / f32 activations" }
                    }
                }
                _ => BackendSupport::Unsupported { reason: "quantised linear takes activation, weight, output" },
            },
            _ => BackendSupport::Unsupported { reason: "the CUDA backend serves the quantised linear op only" },
        }
    }

    fn materialize(&self, _view: &TensorView) -> std::result::Result<MaterializedTensor, BackendError> {
        Err(BackendError::BackendUnavailable { name: self.name() })
    }

    /// The trait's `execute` carries no buffers; numerical work goes through `submit_linear`.
    fn execute(&self, _operation: &SemanticOp) -> std::result::Result<ExecutionReceipt, BackendError> {
        Err(BackendError::BackendUnavailable { name: self.name() })
    }
}

#[cfg(test)]
mod tests {
    use super::*;

    #[test]
    fn status_round_trips() {
        for raw in 0..=17 {
            assert_eq!(Status::from_raw(raw).raw(), raw);
        }
        assert_eq!(Status::from_raw(99), Status::Unknown(99));
    }

    #[test]
    fn abi_version_is_one_and_the_library_never_falls_back() {
        assert_eq!(abi_version().unwrap(), 1);
        let probe = backend_probe().unwrap();
        if !probe.available {
            // no CPU fallback: connecting fails loudly (crates/ullm-hip/src/lib.rs:668-675 checks the same of the stub)
            assert_eq!(CudaBackend::connect(0).err().unwrap().status, Status::CudaUnavailable);
        }
    }
}

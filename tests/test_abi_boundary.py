"""CPU tests of the C-ABI boundary: every declared symbol is exported, struct
layouts match the header, and the error-sink / validation behaviour reproduces
the reference's known answers (crates/ullm-hip/src/lib.rs:677-742, :774-956).
No compute call is made; without a GPU every device entry must answer
CUDA_UNAVAILABLE — never run on the CPU (crates/ullm-hip/src/lib.rs:668-675)."""
import ctypes as C
import os
import re

import pytest

import ullm_cuda as U
from ullm_cuda import _abi as abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
UNAVAILABLE_TEXT = "CUDA backend is unavailable: no usable device; no CPU fallback exists"


def header_functions():
    text = open(os.path.join(ROOT, "include", "ullm_cuda.h")).read()
    return sorted(set(re.findall(r"ULLM_CUDA_API ullm_status_t (ullm_cuda_\w+)\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = abi.load()
    names = header_functions()
    assert len(names) >= 40
    assert sorted(abi.SIGNATURES) == names  # the binding declares exactly the header's functions
    for n in names:
        assert getattr(lib, n) is not None


def test_struct_layouts_match_the_header_pins():
    text = open(os.path.join(ROOT, "include", "ullm_cuda.h")).read()
    pins = dict(re.findall(r"static_assert\(sizeof\((\w+)\) == (\d+)U", text))
    by_name = {"ullm_cuda_error_sink_t": abi.ErrorSink, "ullm_cuda_version_info_t": abi.VersionInfo,
               "ullm_cuda_backend_probe_result_t": abi.BackendProbeResult,
               "ullm_cuda_context_probe_result_t": abi.ContextProbeResult, "ullm_cuda_tensor_t": abi.Tensor,
               "ullm_cuda_weight_t": abi.Weight, "ullm_cuda_completion_result_t": abi.CompletionResult,
               "ullm_cuda_linear_desc_t": abi.LinearDesc, "ullm_cuda_stack_desc_t": abi.StackDesc,
               "ullm_cuda_stack_linear_info_t": abi.StackLinearInfo, "ullm_cuda_slots_t": abi.Slots,
               "ullm_cuda_plan_op_t": abi.PlanOp, "ullm_cuda_binding_t": abi.Binding,
               "ullm_cuda_safetensors_info_t": abi.SafetensorsInfo}
    assert set(pins) == set(by_name)
    for name, cls in by_name.items():
        assert C.sizeof(cls) == int(pins[name]) == abi.EXPECTED_SIZES[cls], name
    assert abi.ErrorSink.message.offset == 8 and abi.ErrorSink.message_capacity.offset == 16
    assert abi.ErrorSink.message_length.offset == 24 and abi.ErrorSink.reserved.offset == 32
    assert abi.LinearDesc.m.offset == 64 and abi.LinearDesc.input.offset == 72 and abi.LinearDesc.output.offset == 96


def test_version_is_abi1_0_1_0():
    assert U.abi_version() == 1
    assert U.version() == U.Version(1, 0, 1, 0)  # crates/ullm-hip/src/lib.rs:756-767


def test_status_mapping_including_unknown_codes():
    assert U.Status.from_raw(0) is U.Status.Ok and U.Status.from_raw(4) is U.Status.CudaUnavailable
    assert U.Status.from_raw(8) is U.Status.Timeout and U.Status.from_raw(12) is U.Status.DispatchContract
    assert U.Status.from_raw(999) is U.Status.Unknown  # crates/ullm-hip/src/lib.rs:562-577


def _probe(sink):
    r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult), abi_version=1)
    return abi.load().ullm_cuda_backend_probe(abi.BACKEND_CUDA, C.byref(r), sink), r


def _sink_for(buf, capacity):
    s = abi.ErrorSink(struct_size=48, abi_version=1)
    s.message = C.cast(buf, C.c_void_p) if buf is not None else None
    s.message_capacity = capacity
    return s


needs_no_gpu = pytest.mark.skipif(U.backend_probe().cuda_runtime_present, reason="asserts the no-device answers")


@needs_no_gpu
def test_error_sink_truncation_known_answers():
    """capacity 1 -> BUFFER_TOO_SMALL, message_length = full length, buffer = [0];
    capacity 0 likewise; exact fit -> primary status; null message with capacity ->
    INVALID_ARGUMENT; null sink -> primary status (crates/ullm-hip/src/lib.rs:918-956)."""
    expected = UNAVAILABLE_TEXT.encode()
    short = C.create_string_buffer(b"\xa5", 1)
    s = _sink_for(short, 1)
    raw, _ = _probe(C.byref(s))
    assert raw == abi.BUFFER_TOO_SMALL and s.message_length == len(expected) and short.raw == b"\x00"
    s = _sink_for(None, 0)
    raw, _ = _probe(C.byref(s))
    assert raw == abi.BUFFER_TOO_SMALL and s.message_length == len(expected)
    full = C.create_string_buffer(len(expected) + 1)
    s = _sink_for(full, len(expected) + 1)
    raw, r = _probe(C.byref(s))
    assert raw == abi.CUDA_UNAVAILABLE and s.message_length == len(expected) and full.value == expected
    assert r.available == 0 and r.backend == abi.BACKEND_CUDA
    s = _sink_for(full, len(expected) + 1)
    s.message = None
    raw, _ = _probe(C.byref(s))
    assert raw == abi.INVALID_ARGUMENT
    raw, _ = _probe(None)
    assert raw == abi.CUDA_UNAVAILABLE


def test_sink_is_validated_before_anything_else_and_without_a_message():
    buf = C.create_string_buffer(b"\xa5" * 64, 64)
    for field, value, want in (("struct_size", 47, abi.INVALID_ARGUMENT), ("abi_version", 2, abi.INVALID_ABI_VERSION)):
        s = _sink_for(buf, 64)
        setattr(s, field, value)
        raw = abi.load().ullm_cuda_backend_probe(999, None, C.byref(s))  # other arguments are wrong too
        assert raw == want and buf.raw == b"\xa5" * 64  # untouched: native/hip/src/hip_stub.cpp:43-66
    s = _sink_for(buf, 64)
    s.reserved[1] = 1
    assert abi.load().ullm_cuda_backend_probe(999, None, C.byref(s)) == abi.RESERVED_NONZERO


def test_struct_validation_order_and_messages():
    lib = abi.load()
    s, buf = U._sink()
    assert lib.ullm_cuda_backend_probe(abi.BACKEND_CUDA, None, C.byref(s)) == abi.INVALID_ARGUMENT
    assert b"null" in buf.value
    r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult) - 1, abi_version=1)
    s, buf = U._sink()
    assert lib.ullm_cuda_backend_probe(abi.BACKEND_CUDA, C.byref(r), C.byref(s)) == abi.INVALID_ARGUMENT
    assert b"struct_size" in buf.value
    r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult), abi_version=2)
    assert lib.ullm_cuda_backend_probe(abi.BACKEND_CUDA, C.byref(r), None) == abi.INVALID_ABI_VERSION
    r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult), abi_version=1)
    r.reserved[2] = 7
    assert lib.ullm_cuda_backend_probe(abi.BACKEND_CUDA, C.byref(r), None) == abi.RESERVED_NONZERO
    r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult), abi_version=1)
    s, buf = U._sink()
    assert lib.ullm_cuda_backend_probe(999, C.byref(r), C.byref(s)) == abi.UNSUPPORTED
    assert b"unknown backend" in buf.value and r.backend == 0  # crates/ullm-hip/src/lib.rs:958-967
    v = abi.VersionInfo(struct_size=C.sizeof(abi.VersionInfo), abi_version=1)
    v.reserved[0] = 1
    assert lib.ullm_cuda_query_version(C.byref(v), None) == abi.RESERVED_NONZERO
    assert lib.ullm_cuda_get_abi_version(None, None) == abi.INVALID_ARGUMENT


@needs_no_gpu
def test_no_device_means_unavailable_never_a_cpu_path():
    with pytest.raises(U.CudaError) as e:
        U.Context(0)
    assert e.value.status is U.Status.CudaUnavailable and "no CPU fallback" in e.value.message
    p = U.backend_probe()
    assert not p.available and "no CPU fallback" in p.diagnostic


def test_stale_and_null_handles_are_rejected_not_dereferenced():
    lib = abi.load()
    bogus = C.c_void_p(0x1234)
    s, buf = U._sink()
    assert lib.ullm_cuda_queue_create(bogus, C.byref(C.c_void_p()), C.byref(s)) == abi.CUDA_INVALID_HANDLE
    assert lib.ullm_cuda_buffer_alloc(None, 16, C.byref(C.c_void_p()), None) == abi.CUDA_INVALID_HANDLE
    assert lib.ullm_cuda_completion_wait(bogus, 0, None, None) == abi.CUDA_INVALID_HANDLE
    assert lib.ullm_cuda_queue_signal(bogus, C.byref(C.c_void_p()), None) == abi.CUDA_INVALID_HANDLE
    h = C.c_void_p(0x1234)
    assert lib.ullm_cuda_buffer_free(C.byref(h), None) == abi.CUDA_INVALID_HANDLE
    assert lib.ullm_cuda_stack_destroy(C.byref(h), None) == abi.CUDA_INVALID_HANDLE
    r = abi.ContextProbeResult(struct_size=C.sizeof(abi.ContextProbeResult), abi_version=1)
    assert lib.ullm_cuda_context_probe(None, C.byref(r), None) == abi.CUDA_UNAVAILABLE
    assert r.context_present == 0 and r.cuda_available == 0


def _desc(enc=abi.ENCODING_AQ4, n=4096, k=4096, m=1, **kw):
    w = abi.Weight(enc, 128 if enc == abi.ENCODING_AQ4 else 0, n, k, abi.Tensor(None, 0), abi.Tensor(None, 0))
    return U.linear_desc(w, m, abi.Tensor(None, 0), abi.Tensor(None, 0), **kw)


def test_linear_supports_answers_from_shape_alone():
    """Mirrors Backend::supports (crates/ullm-core/src/backend.rs:8): no device needed."""
    assert U.linear_supports(_desc()) == abi.KERNEL_MATVEC
    # the same answers with or without a device or driver: a shape query never asks either
    assert U.linear_supports(_desc(abi.ENCODING_FP8_CHANNEL, 14336, 4096, 8)) == abi.KERNEL_GEMM
    assert U.linear_supports(_desc(abi.ENCODING_FP8_CHANNEL, 14336, 4096, 1)) == abi.KERNEL_MATVEC
    assert U.linear_supports(_desc(abi.ENCODING_AQ4, 14336, 4096, 4)) == abi.KERNEL_MATVEC
    assert U.linear_supports(_desc(abi.ENCODING_AQ4, 14336, 4096, 2048)) == abi.KERNEL_GEMM
    assert U.linear_supports(_desc(abi.ENCODING_FP8_CHANNEL, 4096, 4112, 4)) == abi.KERNEL_MATVEC  # K % 128 != 0
    for bad, status in ((_desc(k=4000), U.Status.Unsupported),  # ragged K is rejected, not guessed
                        (_desc(abi.ENCODING_NVFP4), U.Status.Unsupported),
                        (_desc(m=0), U.Status.InvalidArgument),
                        (_desc(input_dtype=abi.DTYPE_U8), U.Status.Unsupported),
                        (_desc(prologue=9), U.Status.InvalidArgument),
                        (_desc(input_row_stride=100), U.Status.InvalidArgument),
                        (_desc(m=5, input_row_stride=1 << 62), U.Status.OutOfRange),  # a span that would wrap 64 bits
                        (_desc(m=5, output_row_stride=(1 << 40) + 1), U.Status.OutOfRange),
                        (_desc(epilogue=abi.EPILOGUE_SWIGLU, residual=abi.Tensor(C.c_void_p(1), 0)), U.Status.Unsupported),
                        (_desc(norm_weight=abi.Tensor(C.c_void_p(1), 0)), U.Status.InvalidArgument)):
        with pytest.raises(U.CudaError) as e:
            U.linear_supports(bad)
        assert e.value.status is status, e.value
    d = _desc()
    d.reserved[0] = 1
    with pytest.raises(U.CudaError) as e:
        U.linear_supports(d)
    assert e.value.status is U.Status.ReservedNonzero
    d = _desc()
    d.abi_version = 3
    with pytest.raises(U.CudaError) as e:
        U.linear_supports(d)
    assert e.value.status is U.Status.InvalidAbiVersion


def test_header_compiles_as_c_and_cxx(tmp_path):
    """native/hip/src/header_c_compile.c / header_cpp_compile.cpp do the same for hip.h."""
    import subprocess
    src = '#include "ullm_cuda.h"\nint main(void){ullm_cuda_error_sink_t s; (void)s; return (int)ULLM_CUDA_ABI_VERSION - 1;}\n'
    for ext, cc, std in ((".c", "gcc", "-std=c99"), (".cpp", "g++", "-std=c++11")):
        f = tmp_path / ("t" + ext)
        f.write_text(src)
        subprocess.run([cc, std, "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
                        str(f), "-o", str(tmp_path / "t.out")], check=True)
        assert subprocess.run([str(tmp_path / "t.out")]).returncode == 0


REF_STUB = os.path.join(ROOT, "oracle", "_ref", "libullm_hip_stub.so")


@needs_no_gpu
@pytest.mark.skipif(not os.path.exists(REF_STUB), reason="reference host stub not built (needs the reference tree)")
def test_sink_behaviour_matches_the_reference_stub_call_for_call():
    """Same calls against the reference's own compiled host stub and this library:
    statuses and sink fields must agree (the message text differs by backend name)."""
    ref = C.CDLL(REF_STUB)

    class RefProbe(C.Structure):
        _fields_ = [("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("backend", C.c_uint32),
                    ("available", C.c_uint32), ("hip_runtime_present", C.c_uint32), ("reserved", C.c_uint32 * 3)]

    def ref_probe(sink, backend=1, mutate=None):
        r = RefProbe(struct_size=C.sizeof(RefProbe), abi_version=1)
        if mutate:
            mutate(r)
        return ref.ullm_backend_probe(backend, C.byref(r), sink)

    def our_probe(sink, backend=abi.BACKEND_CUDA, mutate=None):
        r = abi.BackendProbeResult(struct_size=C.sizeof(abi.BackendProbeResult), abi_version=1)
        if mutate:
            mutate(r)
        return abi.load().ullm_cuda_backend_probe(backend, C.byref(r), sink)

    def bump(field, delta):
        return lambda r: setattr(r, field, getattr(r, field) + delta)

    cases = [dict(), dict(backend=999), dict(mutate=bump("struct_size", -1)), dict(mutate=bump("abi_version", 1)),
             dict(mutate=lambda r: r.reserved.__setitem__(0, 1))]
    for kw in cases:
        for cap in (0, 1, 8, 256):
            b1, b2 = C.create_string_buffer(max(cap, 1)), C.create_string_buffer(max(cap, 1))
            s1, s2 = _sink_for(b1 if cap else None, cap), _sink_for(b2 if cap else None, cap)
            r1, r2 = ref_probe(C.byref(s1), **kw), our_probe(C.byref(s2), **kw)
            assert r1 == r2, (kw, cap, r1, r2)
            assert (s1.message_length > 0) == (s2.message_length > 0)
            if cap:
                assert b1.raw[min(cap - 1, s1.message_length)] == 0 and b2.raw[min(cap - 1, s2.message_length)] == 0
        assert ref_probe(None, **kw) == our_probe(None, **kw)

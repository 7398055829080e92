"""GPU parity of the fused-dequant linear op against the oracle.

Tolerance (stated by the benchmark definition): max relative error 1e-2 and mean
absolute error 1e-3 with fp32 accumulation, evaluated as
max |y-r| / max(|r|, 0.05 rms(r)) <= 1e-2 and mean |y-r| <= 1e-3 (oracle.error_stats)."""
import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, DeviceWeight, oracle_dequantize, oracle_linear, oracle_quantize, run_linear

pytestmark = pytest.mark.gpu
ENCODINGS = [U.ENCODING_AQ4, U.ENCODING_FP8_CHANNEL]


def check(y, ref, what=""):
    st = o.error_stats(y, ref)
    assert st["pass"], (what, st)
    return st


def check_norm(y, ref, what=""):
    """For outputs behind an RMSNorm: the device normalises in fp32, the oracle in fp64, so a handful of normalised
    activations round to the neighbouring bf16 value and move an output that sits on a rounding boundary by one
    more ulp.  Mean error and NaN classes as everywhere; a few element-wise outliers are allowed."""
    st = o.error_stats(y, ref)
    assert st["nan"] == 0 and st["inf"] == 0 and st["mean_abs"] <= 1e-3 and st["max_rel_floored"] <= 2e-2 and \
        st["outliers"] <= max(2, st["n"] // 2000), (what, st)
    return st


# boundary sets: N over tile/warp-group edges, K over piece/iteration edges, every M the matvec serves
CASES = [(1, 1, 128), (1, 3, 256), (2, 17, 384), (3, 255, 1024), (4, 256, 1152), (5, 257, 2048),
         (7, 73, 4096), (8, 37, 3584), (1, 4096, 4096), (8, 1024, 4096), (1, 613, 14336), (3, 64, 14336)]


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("m,n,k", CASES)
def test_matvec_matches_oracle(gpu, encoding, m, n, k):
    ctx, q = gpu
    w = o.synth_weights(SEED, 500 + n + k, n, k)
    x = o.synth_activations(SEED, 600 + m + k, m, k)
    dw = DeviceWeight(ctx, q, w, encoding)
    v, s = oracle_quantize(w, encoding)
    assert np.array_equal(dw.download(q)[0], v)
    ref = oracle_linear(x, oracle_dequantize(v, s, encoding))
    y, res = run_linear(ctx, q, dw, x, kernel=U.KERNEL_MATVEC)
    check(y, ref, (encoding, m, n, k))
    assert res.dispatch_count >= 1 and res.selected_backend == 2 and res.fallback_used == 0 and res.device_flags == 0
    # fp32 output before the bf16 rounding: compare against the unrounded oracle, much tighter
    yf, _ = run_linear(ctx, q, dw, x, kernel=U.KERNEL_MATVEC, y_dtype=U.DTYPE_F32)
    ref64 = oracle_linear(x, oracle_dequantize(v, s, encoding), out="f64")
    scale = np.abs(ref64).max() + 1e-30
    assert np.abs(yf - ref64).max() / scale < 2e-5, np.abs(yf - ref64).max() / scale
    assert dw.canaries_intact(q)
    dw.close()


@pytest.mark.parametrize("encoding", ENCODINGS)
def test_golden_outputs(gpu, golden, encoding):
    ctx, q = gpu
    key = "aq4" if encoding == U.ENCODING_AQ4 else "fp8"
    for name, tw, m, n, k in (("a", 11, 1, 17, 256), ("b", 13, 3, 37, 384), ("c", 15, 8, 73, 1024)):
        dw = DeviceWeight(ctx, q, o.planted_case_weights(SEED, tw, n, k), encoding)
        x = o.bf16_bits_to_f32(golden[f"{name}_x_bits"])
        y, _ = run_linear(ctx, q, dw, x)
        check(y, o.bf16_bits_to_f32(golden[f"{name}_y_{key}_bits"]), name)
        dw.close()


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("prologue", [U.PROLOGUE_RMSNORM, U.PROLOGUE_SWIGLU])
@pytest.mark.parametrize("x_dtype", [U.DTYPE_BF16, U.DTYPE_F32])
def test_prologues_and_dtypes(gpu, encoding, prologue, x_dtype):
    ctx, q = gpu
    m, n, k = 3, 129, 1024
    cols = 2 * k if prologue == U.PROLOGUE_SWIGLU else k
    w = o.synth_weights(SEED, 700, n, k)
    xs = o.synth_normal(SEED, 701, 0, m * cols).reshape(m, cols) * np.float32(1.7)
    x = xs if x_dtype == U.DTYPE_F32 else o.bf16_round(xs)
    dw = DeviceWeight(ctx, q, w, encoding)
    v, s = oracle_quantize(w, encoding)
    ref = oracle_linear(x, oracle_dequantize(v, s, encoding), prologue, x_is_f32=x_dtype == U.DTYPE_F32)
    y, _ = run_linear(ctx, q, dw, x, x_dtype=x_dtype, prologue=prologue)
    check(y, ref, (encoding, prologue, x_dtype))
    dw.close()


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("m,n,k,epilogue", [(1, 10240, 1024, U.EPILOGUE_NONE), (1, 14336, 4096, U.EPILOGUE_NONE),
                                            (1, 9600, 512, U.EPILOGUE_NONE), (1, 9473, 1536, U.EPILOGUE_NONE),
                                            (2, 5000, 1024, U.EPILOGUE_NONE), (4, 4800, 2560, U.EPILOGUE_NONE),
                                            (1, 19200, 512, U.EPILOGUE_SWIGLU), (1, 19000, 2048, U.EPILOGUE_SWIGLU)])
def test_matvec_more_row_groups_than_warps(gpu, encoding, m, n, k, epilogue):
    """Matrices with a little more than a whole number of rounds of row groups over the GPU's warps: the FP8 kernel
    cuts the left-over groups into K slices taken by several warps (slices with and without work, odd row counts,
    the paired rows of the SwiGLU epilogue); the result must not depend on it."""
    ctx, q = gpu
    w = o.synth_weights(SEED, 2500 + n + k, n, k)
    x = o.synth_activations(SEED, 2600 + m + k, m, k)
    dw = DeviceWeight(ctx, q, w, encoding)
    wdq = oracle_dequantize(*oracle_quantize(w, encoding), encoding)
    ref = oracle_linear(x, wdq, epilogue=epilogue)
    y, res = run_linear(ctx, q, dw, x, kernel=U.KERNEL_MATVEC, epilogue=epilogue)
    check(y, ref, (encoding, m, n, k))
    assert res.device_flags == 0 and res.fallback_used == 0
    if epilogue == U.EPILOGUE_NONE:
        yf, _ = run_linear(ctx, q, dw, x, kernel=U.KERNEL_MATVEC, y_dtype=U.DTYPE_F32)
        ref64 = oracle_linear(x, wdq, out="f64")
        assert np.abs(yf - ref64).max() <= 2e-5 * (np.abs(ref64).max() + 1e-30)
        # the same launch twice gives the same bits (fixed summation order across the slices)
        yf2, _ = run_linear(ctx, q, dw, x, kernel=U.KERNEL_MATVEC, y_dtype=U.DTYPE_F32)
        assert np.array_equal(yf.view(np.uint32), yf2.view(np.uint32))
    assert dw.canaries_intact(q)
    dw.close()


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("m,n,k", [(1, 2, 128), (1, 1030, 1024), (2, 514, 512), (4, 256, 1024), (8, 70, 2048)])
def test_swiglu_epilogue(gpu, encoding, m, n, k):
    """Rows [gate(N/2) | up(N/2)] -> [M, N/2] = bf16(silu(bf16 g) * bf16 u)."""
    ctx, q = gpu
    w = o.synth_weights(SEED, 740 + n, n, k) * np.float32(3.0)
    x = o.synth_activations(SEED, 741 + m, m, k)
    dw = DeviceWeight(ctx, q, w, encoding)
    v, s = oracle_quantize(w, encoding)
    ref = oracle_linear(x, oracle_dequantize(v, s, encoding), epilogue=U.EPILOGUE_SWIGLU)
    y, _ = run_linear(ctx, q, dw, x, epilogue=U.EPILOGUE_SWIGLU, kernel=U.KERNEL_MATVEC)
    assert y.shape == (m, n // 2)
    check(y, ref, (encoding, m, n, k))
    y2, _ = run_linear(ctx, q, dw, x, epilogue=U.EPILOGUE_SWIGLU, y_stride=n // 2 + 6)
    check(y2, ref)
    dw.close()


@pytest.mark.parametrize("encoding", ENCODINGS)
def test_strided_rows_and_enqueue_path(gpu, encoding):
    ctx, q = gpu
    m, n, k = 4, 96, 512
    w = o.synth_weights(SEED, 710, n, k)
    x = o.synth_activations(SEED, 711, m, k)
    dw = DeviceWeight(ctx, q, w, encoding)
    v, s = oracle_quantize(w, encoding)
    ref = oracle_linear(x, oracle_dequantize(v, s, encoding))
    y, _ = run_linear(ctx, q, dw, x, x_stride=k + 64, y_stride=n + 32, submit=False)
    check(y, ref)
    dw.close()


def test_linearity_and_zero_input(gpu):
    """Size-independent properties: zero in -> zero out; y(2x) = 2 y(x) exactly in fp32 output."""
    ctx, q = gpu
    m, n, k = 2, 300, 2048
    for encoding in ENCODINGS:
        dw = DeviceWeight(ctx, q, o.synth_weights(SEED, 720, n, k), encoding)
        x = o.synth_activations(SEED, 721, m, k)
        y0, _ = run_linear(ctx, q, dw, np.zeros_like(x), y_dtype=U.DTYPE_F32)
        assert not y0.any()
        y1, _ = run_linear(ctx, q, dw, x, y_dtype=U.DTYPE_F32)
        y2, _ = run_linear(ctx, q, dw, 2 * x, y_dtype=U.DTYPE_F32)
        assert np.allclose(y2, 2 * y1, rtol=1e-5, atol=1e-6)
        dw.close()


def test_full_size_configs_on_sampled_rows(gpu):
    """The benchmark shapes at full size: AQ4 M=1 K=N=4096 and FP8 M in {1,4,8} K=4096 N=14336,
    generated and quantised on the device, checked on a strided sample of output rows."""
    ctx, q = gpu
    for encoding, n, k, ms in ((U.ENCODING_AQ4, 4096, 4096, (1,)), (U.ENCODING_FP8_CHANNEL, 14336, 4096, (1, 4, 8))):
        src = ctx.alloc(n * k * 4)
        q.synth_weights(SEED, 800 + encoding, 0, n * k, 0.02, src.at(0))
        vb, sb = U.weight_bytes(encoding, n, k)
        vals, scl = ctx.alloc(vb), ctx.alloc(sb)
        wd = U.weight_desc(encoding, n, k, vals.at(0), scl.at(0))
        q.quantize(src.at(0), wd)
        rows = np.arange(0, n, 97)
        wrows = np.stack([o.synth_weights(SEED, 800 + encoding, 1, k, row0=int(r))[0] for r in rows])
        v, s = oracle_quantize(wrows, encoding)
        wdq = oracle_dequantize(v, s, encoding)
        for m in ms:
            x = o.synth_activations(SEED, 810 + m, m, k)
            xb, yb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
            q.upload(xb.at(0), o.f32_to_bf16_bits(x))
            q.linear_submit(U.linear_desc(wd, m, xb.at(0), yb.at(0))).wait()
            y = o.bf16_bits_to_f32(q.download(yb.at(0), (m, n), np.uint16))
            check(y[:, rows], o.linear(x, wdq), (encoding, m))
            xb.close()
            yb.close()
        for b in (src, vals, scl):
            b.close()


def test_completion_contract(gpu):
    """submit -> wait consumes the handle; a second wait is INVALID_HANDLE; timeout 0 is one poll
    (native/hip/src/hip_evidence_runtime.hip.cpp:508-535, :691-698)."""
    ctx, q = gpu
    c = q.signal()
    r = c.wait(1000)
    assert r.terminal == 1 and r.fallback_used == 0 and r.selected_backend == 2
    with pytest.raises(U.CudaError) as e:
        c2 = U.Completion()
        c2._h = U.C.c_void_p(0xdead0)
        c2.wait(0)
    assert e.value.status is U.Status.InvalidHandle
    c3 = q.signal()
    assert c3.query(1000)
    c3.close()


def test_graph_capture_replays_a_linear(gpu):
    ctx, q = gpu
    m, n, k = 1, 256, 1024
    dw = DeviceWeight(ctx, q, o.synth_weights(SEED, 730, n, k), U.ENCODING_FP8_CHANNEL)
    x = o.synth_activations(SEED, 731, m, k)
    xb, yb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
    q.upload(xb.at(0), o.f32_to_bf16_bits(x))
    d = U.linear_desc(dw.desc, m, xb.at(0), yb.at(0))
    q.capture_begin()
    q.linear_enqueue(d)
    g = q.capture_end()
    q.fill(yb.at(0), 0, m * n * 2)
    q.synchronize()  # resets the per-signal dispatch counter
    g.launch(q)
    g.launch(q)
    res = q.synchronize()
    assert res.dispatch_count == 2
    v, s = oracle_quantize(o.synth_weights(SEED, 730, n, k), U.ENCODING_FP8_CHANNEL)
    check(o.bf16_bits_to_f32(q.download(yb.at(0), (m, n), np.uint16)), o.linear(x, o.fp8_dequantize(v, s)))
    g.close()
    for b in (xb, yb):
        b.close()
    dw.close()


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("m,kernel", [(1, U.KERNEL_MATVEC), (3, U.KERNEL_MATVEC), (8, U.KERNEL_GEMM), (40, U.KERNEL_GEMM),
                                      (200, U.KERNEL_GEMM)])
def test_rmsnorm_weight_and_residual(gpu, encoding, m, kernel):
    """The glue of a decoder block around the linear: RMSNorm with a weight vector in front (one rounding:
    bf16(x * rsqrt(mean x^2 + eps) * gamma)) and a residual added to the fp32 result, on both kernels.
    (docs/plans/archive/2026/08/1-10/phase2-h3-g0-model-free-gpu.md:42 lists RMSNorm among the first ops.)"""
    ctx, q = gpu
    n, k = 384, 1024
    w = o.synth_weights(SEED, 2100 + m, n, k)
    dw = DeviceWeight(ctx, q, w, encoding)
    wdq = oracle_dequantize(*oracle_quantize(w, encoding), encoding)
    x = (o.synth_normal(SEED, 2200 + m, 0, m * k).reshape(m, k) * np.float32(3.0)).astype(np.float32)  # fp32 input
    gamma = o.bf16_round((1.0 + 0.25 * o.synth_normal(SEED, 2300, 0, k)).astype(np.float32))
    res = (o.synth_normal(SEED, 2400 + m, 0, m * n).reshape(m, n) * np.float32(2.0)).astype(np.float32)
    for out, ydt in (("f32", U.DTYPE_F32), ("bf16", U.DTYPE_BF16)):
        y, _ = run_linear(ctx, q, dw, x, x_dtype=U.DTYPE_F32, y_dtype=ydt, prologue=U.PROLOGUE_RMSNORM, kernel=kernel,
                          gamma=gamma, residual=res)
        ref = oracle_linear(x, wdq, U.PROLOGUE_RMSNORM, x_is_f32=True, out=out, gamma=gamma, residual=res)
        check_norm(y, ref, (encoding, m, kernel, out))
    # the weight vector alone, and the residual alone (in place: the residual aliases the output)
    y, _ = run_linear(ctx, q, dw, x, x_dtype=U.DTYPE_F32, prologue=U.PROLOGUE_RMSNORM, kernel=kernel, gamma=gamma)
    check_norm(y, oracle_linear(x, wdq, U.PROLOGUE_RMSNORM, x_is_f32=True, gamma=gamma), "gamma only")
    xb = o.bf16_round(x)
    ybuf, xbuf = ctx.alloc(m * n * 4), ctx.alloc(m * k * 2)
    q.upload(ybuf.at(0), res)
    q.upload(xbuf.at(0), o.f32_to_bf16_bits(xb).reshape(m, k))
    q.linear_submit(U.linear_desc(dw.desc, m, xbuf.at(0), ybuf.at(0), output_dtype=U.DTYPE_F32, kernel=kernel,
                                  residual=ybuf.at(0))).wait(60000)
    y = q.download(ybuf.at(0), (m, n), np.float32)
    check(y, oracle_linear(xb, wdq, out="f32", residual=res), "in-place residual")
    ybuf.close()
    xbuf.close()
    dw.close()

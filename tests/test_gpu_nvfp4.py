"""NVFP4 (e2m1 values, blocks of 16, f16 block scales, one f32 tensor scale — the packed 4-bit descriptor the reference
defines in crates/ullm-core/src/dtype.rs:56-66 with the tensor scale its plan adds, docs/plans/main-plan.md:102-114):
quantise / dequantise bit-exact against the oracle, and the decode linear at the stated tolerance."""
import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, oracle_linear

pytestmark = pytest.mark.gpu
ENC = U.ENCODING_NVFP4


def _device_weight(ctx, q, w):
    n, k = w.shape
    vb, sb = U.weight_bytes(ENC, n, k)
    src, vals, scl = ctx.alloc(w.nbytes), ctx.alloc(vb + 256), ctx.alloc(sb + 256)
    q.fill(vals.at(0), 0xC5, vb + 256)
    q.fill(scl.at(0), 0xC5, sb + 256)
    q.upload(src.at(0), w)
    wd = U.weight_desc(ENC, n, k, vals.at(0), scl.at(0))
    q.quantize(src.at(0), wd)
    return wd, (src, vals, scl), vb, sb


@pytest.mark.parametrize("n,k", [(1, 32), (3, 64), (37, 1024), (257, 4096), (64, 14336)])
def test_quantise_and_dequantise_are_bit_exact(gpu, n, k):
    ctx, q = gpu
    w = o.synth_weights(SEED, 7000 + n + k, n, k)
    if n >= 3:  # planted cases: a zero block, a lone outlier, ties on every midpoint of the e2m1 grid
        w[0, :16] = 0.0
        w[1, 5] = 1.0
        w[2, :16] = np.array([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 5.5], np.float32) * np.float32(0.125)
    wd, bufs, vb, sb = _device_weight(ctx, q, w)
    packed, sbl, ts = o.nvfp4_quantize(w)
    assert o.nvfp4_scale_bytes(n, k) == sb
    assert np.array_equal(q.download(bufs[1].at(0), (n, k // 2), np.uint8), packed)
    assert np.array_equal(q.download(bufs[2].at(0), (n, k // 16), np.float16).view(np.uint16), sbl.view(np.uint16))
    ts_off = (n * (k // 16) * 2 + 15) // 16 * 16
    assert q.download(bufs[2].at(ts_off), (1,), np.float32)[0] == ts
    assert (q.download(bufs[1].at(vb), (256,), np.uint8) == 0xC5).all() and (q.download(bufs[2].at(sb), (256,), np.uint8) == 0xC5).all()
    out = ctx.alloc(n * k * 4)
    q.dequantize(wd, out.at(0), U.DTYPE_F32)
    ref = o.nvfp4_dequantize(packed, sbl, ts)
    assert np.array_equal(q.download(out.at(0), (n, k), np.float32).view(np.uint32), ref.view(np.uint32))
    q.dequantize(wd, out.at(0), U.DTYPE_BF16)
    assert np.array_equal(q.download(out.at(0), (n, k), np.uint16), o.f32_to_bf16_bits(ref).reshape(n, k))
    for b in bufs + (out,):
        b.close()


def test_all_zero_tensor_and_every_code(gpu):
    ctx, q = gpu
    wd, bufs, _, sb = _device_weight(ctx, q, np.zeros((2, 32), np.float32))
    assert (q.download(bufs[1].at(0), (2, 16), np.uint8) == 0).all()
    assert q.download(bufs[2].at((2 * 2 * 2 + 15) // 16 * 16), (1,), np.float32)[0] == 1.0
    for b in bufs:
        b.close()
    # every code 0..15 decodes to the oracle's value (negative zero, code 8, included)
    codes = np.arange(16, dtype=np.uint8)
    packed = (codes[0::2] | (codes[1::2] << 4)).reshape(1, 8)
    packed = np.concatenate([packed, packed], axis=1)  # 32 values
    vals, scl, out = ctx.alloc(16), ctx.alloc(32), ctx.alloc(32 * 4)
    q.upload(vals.at(0), packed)
    sc = np.zeros(16, np.uint8)
    sc[:4] = np.array([1.5, 0.75], np.float16).view(np.uint8)
    q.upload(scl.at(0), sc)
    q.upload(scl.at(16), np.array([0.25], np.float32))
    wd = U.weight_desc(ENC, 1, 32, vals.at(0), scl.at(0))
    q.dequantize(wd, out.at(0), U.DTYPE_F32)
    got = q.download(out.at(0), (1, 32), np.float32)
    want = o.nvfp4_dequantize(packed, np.array([[1.5, 0.75]], np.float16), np.float32(0.25))
    assert np.array_equal(got, want)
    for b in (vals, scl, out):
        b.close()


@pytest.mark.parametrize("m,n,k", [(1, 1, 32), (1, 257, 1024), (2, 73, 4096), (5, 130, 2080), (8, 64, 4096), (1, 2048, 14336), (3, 40, 8192)])
def test_decode_linear_matches_the_oracle(gpu, m, n, k):
    ctx, q = gpu
    w = o.synth_weights(SEED, 7100 + n + k, n, k)
    wd, bufs, _, _ = _device_weight(ctx, q, w)
    wdq = o.nvfp4_dequantize(*o.nvfp4_quantize(w))
    x = o.synth_activations(SEED, 7200 + m + k, m, k)
    res = (o.synth_normal(SEED, 7300 + m, 0, m * n).reshape(m, n)).astype(np.float32)
    xb, yb, rb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 4 + 256), ctx.alloc(m * n * 4)
    q.upload(xb.at(0), o.f32_to_bf16_bits(x).reshape(m, k))
    q.upload(rb.at(0), res)
    assert U.linear_supports(U.linear_desc(wd, m, xb.at(0), yb.at(0))) == U.KERNEL_MATVEC
    r = q.linear_submit(U.linear_desc(wd, m, xb.at(0), yb.at(0))).wait(60000)
    assert r.device_flags == 0 and r.fallback_used == 0
    y = o.bf16_bits_to_f32(q.download(yb.at(0), (m, n), np.uint16))
    st = o.error_stats(y, oracle_linear(x, wdq))
    assert st["pass"], st
    q.fill(yb.at(0), 0xC5, m * n * 4 + 256)
    q.linear_submit(U.linear_desc(wd, m, xb.at(0), yb.at(0), output_dtype=U.DTYPE_F32, residual=rb.at(0))).wait(60000)
    yf = q.download(yb.at(0), (m, n), np.float32)
    ref64 = oracle_linear(x, wdq, out="f64") + res.astype(np.float64)
    assert np.abs(yf - ref64).max() <= 2e-5 * (np.abs(ref64).max() + 1e-30)
    assert (q.download(yb.at(m * n * 4), (256,), np.uint8) == 0xC5).all()
    for b in bufs + (xb, yb, rb):
        b.close()


def test_what_nvfp4_does_not_offer_is_answered_not_guessed(gpu):
    ctx, q = gpu
    none = U.abi.Tensor(None, 0)
    w = U.abi.Weight(ENC, 16, 256, 1024, none, none)
    assert U.linear_supports(U.linear_desc(w, 8, none, none)) == U.KERNEL_MATVEC
    for d in (U.linear_desc(w, 9, none, none),                                   # no tensor-core path
              U.linear_desc(w, 1, none, none, kernel=U.KERNEL_GEMM),
              U.linear_desc(w, 1, none, none, prologue=U.PROLOGUE_RMSNORM),
              U.linear_desc(w, 1, none, none, epilogue=U.EPILOGUE_SWIGLU),
              U.linear_desc(U.abi.Weight(ENC, 16, 256, 1000, none, none), 1, none, none),   # K % 32
              U.linear_desc(U.abi.Weight(ENC, 32, 256, 1024, none, none), 1, none, none)):  # block size
        with pytest.raises(U.CudaError) as e:
            U.linear_supports(d)
        assert e.value.status is U.Status.Unsupported, e.value

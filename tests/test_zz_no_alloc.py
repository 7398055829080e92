"""The allocation-free linear entry point (staging area = a fixed device array inside the library)
gives the same result as the regular entry point, twice in a row.

Collected last on purpose: if it fails under `pytest -x`, every other test has already run.
It must pass both in a fresh process and after the rest of the suite (the array is shared by all
calls and keeps the previous call's contents, so the second call starts from a dirty array)."""
import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, DeviceWeight, oracle_dequantize, oracle_linear, oracle_quantize

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("encoding", [U.ENCODING_FP8_CHANNEL, U.ENCODING_AQ4])
def test_static_scratch_entry_matches_the_regular_one(gpu, encoding):
    ctx, q = gpu
    m, n, k = 48, 384, 1024
    w = o.synth_weights(SEED, 2100, n, k)
    x = (o.synth_normal(SEED, 2101, 0, m * k).reshape(m, k) * np.float32(1.5)).astype(np.float32)  # fp32 in, RMSNorm prologue
    dw = DeviceWeight(ctx, q, w, encoding)
    xb, y_ref, y_new = ctx.alloc(x.nbytes), ctx.alloc(m * n * 2), ctx.alloc(m * n * 2)
    q.upload(xb.at(0), x)
    kw = dict(input_dtype=U.DTYPE_F32, prologue=U.PROLOGUE_RMSNORM, kernel=U.KERNEL_GEMM)
    q.linear_enqueue(U.linear_desc(dw.desc, m, xb.at(0), y_ref.at(0), **kw))
    q.synchronize()
    ref_bits = q.download(y_ref.at(0), (m, n), np.uint16)
    v, s = oracle_quantize(w, encoding)
    oracle = oracle_linear(x, oracle_dequantize(v, s, encoding), U.PROLOGUE_RMSNORM, x_is_f32=True)
    assert o.error_stats(o.bf16_bits_to_f32(ref_bits), oracle)["pass"]
    # The regular entry point may cut a tile's K range over several CTAs and add fp32 partials; the
    # allocation-free one has no room for partials and gives every CTA whole tiles.  Same products, another
    # order of fp32 additions: the bf16 outputs agree except where a sum sits on a rounding boundary.
    first = None
    for attempt in range(2):  # the second call finds the previous call's data in the shared array
        q.fill(y_new.at(0), 0xC5, m * n * 2)
        q.linear_enqueue_static_scratch(U.linear_desc(dw.desc, m, xb.at(0), y_new.at(0), **kw))
        res = q.synchronize()
        assert res.device_flags == 0
        got = q.download(y_new.at(0), (m, n), np.uint16)
        st = o.error_stats(o.bf16_bits_to_f32(got), o.bf16_bits_to_f32(ref_bits))
        ulps = np.abs(got.astype(np.int32) - ref_bits.astype(np.int32))
        assert st["pass"] and ulps.max() <= 1 and (ulps == 0).mean() >= 0.99, (attempt, st, int(ulps.max()))
        assert o.error_stats(o.bf16_bits_to_f32(got), oracle)["pass"]
        if first is None:
            first = got
        assert np.array_equal(got, first)  # call after call: bit-identical
    # a different (smaller) problem right after reuses the same array
    m2 = 9
    q.linear_enqueue_static_scratch(U.linear_desc(dw.desc, m2, xb.at(0), y_new.at(0), **kw))
    q.linear_enqueue(U.linear_desc(dw.desc, m2, xb.at(0), y_ref.at(0), **kw))
    q.synchronize()
    a9, b9 = q.download(y_new.at(0), (m2, n), np.uint16), q.download(y_ref.at(0), (m2, n), np.uint16)
    assert np.abs(a9.astype(np.int32) - b9.astype(np.int32)).max() <= 1
    for b in (xb, y_ref, y_new):
        b.close()
    dw.close()


def test_static_scratch_entry_rejects_what_does_not_fit(gpu):
    ctx, q = gpu
    n, k = 128, 8192
    m = U.abi.STATIC_SCRATCH_BYTES // (2 * k) + 1  # one row too many for the fixed array
    dw = DeviceWeight(ctx, q, o.synth_weights(SEED, 2110, n, k), U.ENCODING_FP8_CHANNEL)
    xb, yb = ctx.alloc(m * k * 4), ctx.alloc(m * n * 2)
    with pytest.raises(U.CudaError) as e:
        q.linear_enqueue_static_scratch(U.linear_desc(dw.desc, m, xb.at(0), yb.at(0), input_dtype=U.DTYPE_F32))
    assert e.value.status is U.Status.Unsupported and "staging" in e.value.message
    with pytest.raises(U.CudaError) as e:
        q.linear_enqueue_static_scratch(U.linear_desc(dw.desc, 16, xb.at(0), yb.at(0), epilogue=U.EPILOGUE_SWIGLU))
    assert e.value.status is U.Status.Unsupported
    for b in (xb, yb):
        b.close()
    dw.close()

"""GPU parity: quantise / pack / unpack / dequantise and the synthetic generator
are BIT-EXACT against the oracle (integer / byte work: no tolerance)."""
import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, DeviceWeight, oracle_dequantize, oracle_quantize

pytestmark = pytest.mark.gpu

SHAPES = [(1, 128), (3, 256), (17, 384), (255, 128), (256, 1024), (257, 4096), (73, 14336)]


@pytest.mark.parametrize("encoding", [U.ENCODING_AQ4, U.ENCODING_FP8_CHANNEL])
@pytest.mark.parametrize("n,k", SHAPES)
def test_quantize_and_dequantize_bit_exact(gpu, encoding, n, k):
    ctx, q = gpu
    w = o.planted_case_weights(SEED, 300 + n, n, k) if n >= 3 else o.synth_weights(SEED, 300 + n, n, k)
    dw = DeviceWeight(ctx, q, w, encoding)
    v, s = dw.download(q)
    rv, rs = oracle_quantize(w, encoding)
    assert np.array_equal(v, rv)
    assert np.array_equal(s.view(np.uint8), np.ascontiguousarray(rs).view(np.uint8))
    assert dw.canaries_intact(q)
    out = ctx.alloc(n * k * 4)
    q.dequantize(dw.desc, out.at(0), U.DTYPE_F32)
    d = q.download(out.at(0), (n, k), np.float32)
    ref = oracle_dequantize(rv, rs, encoding)
    assert np.array_equal(d.view(np.uint32), ref.view(np.uint32))
    q.dequantize(dw.desc, out.at(0), U.DTYPE_BF16)
    db = q.download(out.at(0), (n, k), np.uint16)
    assert np.array_equal(db, o.f32_to_bf16_bits(ref).reshape(n, k))
    out.close()
    dw.close()


def test_golden_vectors_on_device(gpu, golden):
    ctx, q = gpu
    for name, tw, n, k in (("a", 11, 17, 256), ("b", 13, 37, 384), ("c", 15, 73, 1024)):
        w = o.planted_case_weights(SEED, tw, n, k)
        for enc, vkey, skey in ((U.ENCODING_AQ4, "aq4_packed", "aq4_scales_bits"),
                                (U.ENCODING_FP8_CHANNEL, "fp8_codes", "fp8_scale")):
            dw = DeviceWeight(ctx, q, w, enc)
            v, s = dw.download(q)
            assert np.array_equal(v, golden[f"{name}_{vkey}"])
            assert np.array_equal(s.view(np.uint8), golden[f"{name}_{skey}"].view(np.uint8))
            dw.close()


def test_aq4_unpack_pack_round_trip(gpu):
    ctx, q = gpu
    n, k = 37, 512
    w = o.synth_weights(SEED, 410, n, k)
    dw = DeviceWeight(ctx, q, w, U.ENCODING_AQ4)
    v, s = dw.download(q)
    qi = ctx.alloc(n * k)
    q.aq4_unpack(dw.desc, qi.at(0))
    ints = q.download(qi.at(0), (n, k), np.int8)
    assert np.array_equal(ints, o.aq4_unpack(v))
    # every code, including 0 (= -8, never produced by the quantiser), survives unpack -> pack
    allcodes = (np.arange(n * k // 2, dtype=np.uint32) % 256).astype(np.uint8).reshape(n, k // 2)
    q.upload(dw.values.at(0), allcodes)
    q.aq4_unpack(dw.desc, qi.at(0))
    ints = q.download(qi.at(0), (n, k), np.int8)
    assert np.array_equal(ints, o.aq4_unpack(allcodes)) and ints.min() == -8 and ints.max() == 7
    q.fill(dw.values.at(0), 0, n * k // 2)
    q.aq4_pack(qi.at(0), dw.desc)
    assert np.array_equal(q.download(dw.values.at(0), (n, k // 2), np.uint8), allcodes)
    with pytest.raises(U.CudaError) as e:  # FP8 has no nibbles to unpack
        fw = DeviceWeight(ctx, q, w, U.ENCODING_FP8_CHANNEL)
        q.aq4_unpack(fw.desc, qi.at(0))
    assert e.value.status is U.Status.Unsupported
    qi.close()
    dw.close()


def test_all_e4m3_codes_decode_exactly(gpu):
    ctx, q = gpu
    codes = np.array([c for c in range(256) if c & 0x7F != 0x7F] * 16, np.uint8)[: 16 * 240].reshape(16, 240)
    vals, scl, out = ctx.alloc(codes.nbytes), ctx.alloc(16 * 4), ctx.alloc(codes.size * 4)
    q.upload(vals.at(0), codes)
    scale = (np.float32(2.0) ** -np.arange(16)).astype(np.float32)
    q.upload(scl.at(0), scale)
    wd = U.weight_desc(U.ENCODING_FP8_CHANNEL, 16, 240, vals.at(0), scl.at(0))
    q.dequantize(wd, out.at(0), U.DTYPE_F32)
    d = q.download(out.at(0), (16, 240), np.float32)
    assert np.array_equal(d, o.fp8_dequantize(codes, scale))
    for b in (vals, scl, out):
        b.close()


def test_generator_matches_oracle_bit_for_bit(gpu):
    ctx, q = gpu
    n = 100_003
    buf = ctx.alloc(n * 4)
    q.synth_weights(SEED, 7, 12345, n, 0.02, buf.at(0))
    assert np.array_equal(q.download(buf.at(0), (n,), np.float32),
                          (o.synth_normal(SEED, 7, 12345, n) * np.float32(0.02)).astype(np.float32))
    q.synth_activations(SEED, 9, 0, n, buf.at(0))
    assert np.array_equal(q.download(buf.at(0), (n,), np.uint16), o.f32_to_bf16_bits(o.synth_normal(SEED, 9, 0, n)))
    buf.close()


def test_spans_are_bounds_checked_on_the_host(gpu):
    ctx, q = gpu
    small = ctx.alloc(1024)
    wd = U.weight_desc(U.ENCODING_AQ4, 64, 128, small.at(0), small.at(0))  # needs 4096 value bytes
    with pytest.raises(U.CudaError) as e:
        q.dequantize(wd, small.at(0), U.DTYPE_F32)
    assert e.value.status is U.Status.OutOfRange
    with pytest.raises(U.CudaError) as e:
        q.upload(small.at(1000), np.zeros(100, np.uint8))
    assert e.value.status is U.Status.OutOfRange
    wd = U.weight_desc(U.ENCODING_AQ4, 4, 130, small.at(0), small.at(0))
    with pytest.raises(U.CudaError) as e:
        q.dequantize(wd, small.at(0), U.DTYPE_F32)
    assert e.value.status is U.Status.Unsupported  # ragged K
    small.close()
    with pytest.raises(U.CudaError) as e:  # freed handle
        q.fill(small.at(0), 0, 4)
    assert e.value.status is U.Status.InvalidHandle

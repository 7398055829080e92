"""CPU tests of the oracle itself: hand-derived known answers, the committed
golden vectors, and NumPy-vs-C agreement.  The reference has no vectors for
this path (parity unpinned), so the known answers below are derived by hand
from the format rules in oracle/oracle.py; the storage-size answers follow the
style of crates/ullm-core/src/lib.rs:98-127."""
import numpy as np
import pytest

import oracle as o
import oracle_c as oc

SEED = o.DEFAULT_SEED
BOUNDARY = [1, 3, 7, 15, 16, 17, 37, 73, 255, 256, 257]  # tests/reference/oracles.py:32-41 (0 handled apart)


def test_storage_bytes_known_answers():
    # N=K=4096: 8,388,608 nibble bytes + 262,144 scale bytes
    assert o.aq4_storage_bytes(4096 * 4096) == 8_388_608 + 262_144
    assert o.aq4_storage_bytes(14336 * 4096) == 29_360_128 + 917_504
    # ragged counts round up like the reference's Nvfp4 descriptor (15 -> 8 + 1 scale)
    assert o.aq4_storage_bytes(15, group=16) == 8 + 2
    assert o.aq4_storage_bytes(17, group=16) == 9 + 4
    # the three answers the reference's own test holds for Nvfp4 { block_size: 16, scale_dtype: F16 }
    # (crates/ullm-core/src/lib.rs:98-127): 15 -> 8 + 2, 16 -> 8 + 2, 17 -> 9 + 4
    assert [o.aq4_storage_bytes(e, group=16) for e in (15, 16, 17)] == [10, 10, 13]
    # NVFP4 as this library lays it out: the same payload and block-scale bytes, the block scales padded to 16 bytes
    # and followed by the f32 tensor scale
    n, k = 24, 64
    rule = o.aq4_storage_bytes(n * k, group=o.NVFP4_BLOCK)
    assert rule == n * k // 2 + n * (k // 16) * 2
    assert o.nvfp4_scale_bytes(n, k) == (rule - n * k // 2 + 15) // 16 * 16 + 4


def test_nibble_and_byte_order():
    q = np.array([[-7, -1, 0, 1, 7, 3, -8, 2]], np.int8)
    p = o.aq4_pack(q)
    # element 2j in the low nibble, 2j+1 in the high nibble; code = q + 8
    assert p.tolist() == [[0x71, 0x98, 0xBF, 0xA0]]
    assert np.array_equal(o.aq4_unpack(p), q)
    assert np.array_equal(oc.aq4_unpack(p), q)


def test_aq4_ties_zero_group_and_outlier():
    w = o.planted_case_weights(SEED, 11, 4, 256)
    p, s = o.aq4_quantize(w)
    q = o.aq4_unpack(p)
    assert s[0, 0] == 0 and (q[0, :128] == 0).all()  # all-zero group -> scale 0, q 0
    assert s[1, 0] == np.float16(1.0 / 7.0) and q[1, 5] == 7  # lone outlier pins the scale
    assert abs(q[1, :128]).sum() == 7 + abs(np.rint(w[1, :128] / np.float32(s[1, 0])))[np.arange(128) != 5].sum()
    assert s[2, 0] == np.float16(1.0)
    assert q[2, :8].tolist() == [7, 0, 2, 2, 0, -2, 6, -6]  # round-half-even
    d = o.aq4_dequantize(p, s)
    assert np.array_equal(d[2, :8], np.array([7, 0, 2, 2, 0, -2, 6, -6], np.float32))


def test_aq4_scale_saturates_and_underflows():
    w = np.zeros((2, 128), np.float32)
    w[0, 0] = 1e9  # amax/7 above the fp16 range -> scale clamps to 65504
    w[1, 0] = 1e-9  # amax/7 below the smallest fp16 subnormal -> scale 0 -> q 0
    p, s = o.aq4_quantize(w)
    assert s[0, 0] == np.float16(65504.0) and o.aq4_unpack(p)[0, 0] == 7
    assert s[1, 0] == 0 and (o.aq4_unpack(p)[1] == 0).all()
    p2, s2 = oc.aq4_quantize(w)
    assert np.array_equal(p, p2) and np.array_equal(s.view(np.uint16), s2.view(np.uint16))


def test_aq4_rejects_ragged_k_and_nonfinite():
    with pytest.raises(ValueError):
        o.aq4_quantize(np.zeros((1, 130), np.float32))
    bad = np.zeros((1, 128), np.float32)
    bad[0, 3] = np.inf
    with pytest.raises(ValueError):
        o.aq4_quantize(bad)
    with pytest.raises(ValueError):
        oc.aq4_quantize(bad)


def test_e4m3_all_codes_round_trip_and_known_values():
    t = o.E4M3_TABLE
    assert t[0x7E] == 448.0 and t[0xFE] == -448.0 and t[0x08] == 2.0 ** -6 and t[0x01] == 2.0 ** -9
    assert np.isnan(t[0x7F]) and np.isnan(t[0xFF])
    codes = np.array([c for c in range(256) if c & 0x7F != 0x7F], np.uint8)
    assert np.array_equal(o.e4m3_encode(t[codes]), codes)
    # saturation and ties: 464 is the midpoint above 448 -> clamps; 0.0146484375 = midway 7*2^-9 / 2^-6
    x = np.array([1000.0, -1000.0, 464.0, 2.0 ** -10, 3 * 2.0 ** -10, 17.0, 19.0], np.float32)
    assert o.e4m3_encode(x).tolist() == [0x7E, 0xFE, 0x7E, 0x00, 0x02, 0x58, 0x5A]


def test_e4m3_encode_matches_ml_dtypes():
    ml = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(SEED)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 0.05, 1.0, 40.0, 300.0)])
    x = np.clip(x, -448, 448)
    assert np.array_equal(o.e4m3_encode(x), x.astype(ml.float8_e4m3fn).view(np.uint8))
    assert np.array_equal(o.f32_to_bf16_bits(x), x.astype(ml.bfloat16).view(np.uint16))


def test_fp8_scale_rule():
    w = o.synth_weights(SEED, 21, 5, 64)
    w[3] = 0.0
    c, s = o.fp8_quantize(w)
    assert np.array_equal(s, (np.abs(w).max(axis=1) / np.float32(448)).astype(np.float32))
    assert s[3] == 0 and (c[3] == 0).all()
    assert (np.abs(o.e4m3_decode(c)).max(axis=1)[[0, 1, 2, 4]] == 448.0).all()  # the row maximum maps to 448


@pytest.mark.parametrize("n", BOUNDARY)
def test_numpy_and_c_agree_on_boundary_shapes(n):
    k = 128 * (1 + n % 3)
    w = o.synth_weights(SEED, 100 + n, n, k)
    p, s = o.aq4_quantize(w)
    p2, s2 = oc.aq4_quantize(w)
    assert np.array_equal(p, p2) and np.array_equal(s.view(np.uint16), s2.view(np.uint16))
    assert np.array_equal(o.aq4_dequantize(p, s), oc.aq4_dequantize(p, s))
    c, cs = o.fp8_quantize(w)
    c2, cs2 = oc.fp8_quantize(w)
    assert np.array_equal(c, c2) and np.array_equal(cs, cs2)
    assert np.array_equal(o.fp8_dequantize(c, cs), oc.fp8_dequantize(c, cs))
    m = 1 + n % 8
    x = o.synth_activations(SEED, 200 + n, m, k)
    xb = oc.synth_activations_bits(SEED, 200 + n, m, k)
    assert np.array_equal(o.f32_to_bf16_bits(x).reshape(m, k), xb)
    for y64, y32 in ((o.linear(x, o.aq4_dequantize(p, s)), oc.linear_aq4(xb, p, s)),
                     (o.linear(x, o.fp8_dequantize(c, cs)), oc.linear_fp8(xb, c, cs))):
        st = o.error_stats(y32, y64)
        assert st["pass"], st


def test_empty_inputs():
    p, s = o.aq4_quantize(np.zeros((0, 128), np.float32))
    assert p.shape == (0, 64) and s.shape == (0, 1)
    assert o.aq4_unpack(p).shape == (0, 128)
    assert o.error_stats(np.zeros(0), np.zeros(0))["pass"]


def test_generator_is_counter_based_and_matches_c():
    a = o.synth_normal(SEED, 7, 0, 4096)
    b = o.synth_normal(SEED, 7, 1000, 96)
    assert np.array_equal(a[1000:1096], b)  # any window can be regenerated on its own
    assert np.array_equal(a, oc.synth_normal(SEED, 7, 0, 4096))
    z = o.synth_normal(SEED, 8, 0, 1 << 18)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01 and np.abs(z).max() < 6.0


def test_golden_vectors(golden):
    cases = [("a", (11, 12), 1, 17, 256), ("b", (13, 14), 3, 37, 384), ("c", (15, 16), 8, 73, 1024)]
    assert np.array_equal(golden["synth_normal_t7_first64"], o.synth_normal(SEED, 7, 0, 64))
    for name, (tw, tx), m, n, k in cases:
        w = o.planted_case_weights(SEED, tw, n, k)
        xb = golden[f"{name}_x_bits"]
        assert np.array_equal(xb, oc.synth_activations_bits(SEED, tx, m, k))
        for impl in (o, oc):
            p, s = impl.aq4_quantize(w)
            c, cs = impl.fp8_quantize(w)
            assert np.array_equal(p, golden[f"{name}_aq4_packed"])
            assert np.array_equal(s.view(np.uint16), golden[f"{name}_aq4_scales_bits"])
            assert np.array_equal(c, golden[f"{name}_fp8_codes"])
            assert np.array_equal(cs, golden[f"{name}_fp8_scale"])
        x = o.bf16_bits_to_f32(xb)
        y = o.f32_to_bf16_bits(o.linear(x, o.aq4_dequantize(golden[f"{name}_aq4_packed"],
                                                            golden[f"{name}_aq4_scales_bits"].view(np.float16))))
        assert np.array_equal(y.reshape(m, n), golden[f"{name}_y_aq4_bits"])
        # fp32-accumulating C port stays inside the stated tolerance of the fp64 golden
        yc = oc.linear_fp8(xb, golden[f"{name}_fp8_codes"], golden[f"{name}_fp8_scale"])
        assert o.error_stats(yc, o.bf16_bits_to_f32(golden[f"{name}_y_fp8_bits"]))["pass"]


def test_error_metric_flags_bad_outputs():
    r = np.linspace(-2, 2, 1001)
    assert o.error_stats(r, r)["pass"]
    bad = r.copy()
    bad[500] += 0.5
    assert not o.error_stats(bad, r)["pass"]
    nan = r.copy()
    nan[3] = np.nan
    st = o.error_stats(nan, r)
    assert st["nan"] == 1 and not st["pass"]

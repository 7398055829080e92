"""CPU oracle for the quantised linear-layer path (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only tests, the smoke check and
the bench's CPU-baseline leg may import it.  The CUDA library must never route
through it.

PARITY UNPINNED.  The reference project (jyohukuchan/uLLM-project) ships no
implementation, golden vector or known-answer test for AQ4 / FP8 quantisation,
packing, matvec or GEMM.  What it does fix, and what this oracle follows:

* packed 4-bit payloads live in ``U8`` storage, ``ceil(n/2)`` bytes, followed by
  one scale per block of consecutive elements, scale dtype in {bf16, f16, f32}
  (crates/ullm-core/src/dtype.rs:56-122, the ``Nvfp4`` descriptor);
* the FP8 flavour is OCP ``e4m3fn`` (no infinities, max finite 448)
  (crates/ullm-core/src/dtype.rs:6-16);
* dtype conversions are bit-exact with stated rounding; float comparisons use
  ``|a-r| <= atol + rtol*|r|`` and report max-abs / max-rel / outliers / NaN
  classes; the oracle states its accumulate dtype and does not copy the kernel's
  control structure (docs/plans/active/2026/08/1-10/ci-test-strategy.md:104-112);
* seeded, bounded boundary sets {0,1,3,7,15,16,17,37,73,255,256,257}, default
  seed 20260803 (tests/reference/oracles.py:16-43).

Everything else (the AQ4 format itself) is specified here, following the
benchmark configuration text: 4-bit symmetric, group of 128 along K, fp16 scale;
FP8 e4m3 with a per-output-channel fp32 scale of amax/448; bf16 activations;
fp32 accumulation; bf16 output.

Format summary (normative for this repository)
----------------------------------------------
AQ4, weight ``W[N,K]`` fp32, ``K % 128 == 0``; for row n and group g:
    amax  = max |w|            over the 128 consecutive k of the group
    scale = fp16_rne(amax / 7) (fp32 division, clamped to 65504)
    q     = 0 if scale == 0 else clamp(rint(w / fp32(scale)), -7, 7)   (rint = ties-to-even)
    u     = q + 8  in [1, 15]  (code 0 never produced; it decodes to -8)
    byte j of the row = u[2j] | u[2j+1] << 4
    layout: packed[N][K/2] u8, then scales[N][K/128] fp16
    dequant w' = fp32(u - 8) * fp32(scale)        (exact in fp32)
FP8, per output channel n:
    scale[n] = fp32(amax_n / 448)  (0 if amax 0)
    w8       = e4m3fn_rne(clamp(w / scale, -448, 448)), 0 if scale == 0
    dequant w' = fp32(w8) * scale[n]              (one fp32 rounding)
NVFP4 (the descriptor the reference defines: crates/ullm-core/src/dtype.rs:56-66, packed 4-bit values with one
scale per block, scale dtype in {bf16, f16, f32}; its plan adds a tensor scale to the tensor representation and the
kernel contract: docs/plans/main-plan.md:102-114).  Here: block 16 along K, f16 block scales, one f32 tensor scale.
    values e2m1 (sign, 2 exponent bits, 1 mantissa bit): magnitudes {0, 0.5, 1, 1.5, 2, 3, 4, 6}
    ts    = 2^floor(log2(amax_tensor / 6))  (a power of two; 1.0 for an all-zero tensor)
    sb    = fp16_rne((amax_block / 6) / ts)             (fp32 divisions)
    code  = 0 if sb == 0 else e2m1_rne(w / (fp32(sb) * ts)), saturating at +-6; ties go to the even code
    byte j of a row = code[2j] | code[2j+1] << 4
    layout: packed[N][K/2] u8; scales: f16 [N][K/16], then (at the next 16-byte boundary) the f32 tensor scale
    dequant w' = e2m1(code) * fp32(sb) * ts             (both products exact in fp32)
Linear:  y[m,n] = bf16_rne( sum_k fp32(x[m,k]) * w'[n,k] ), fp64 accumulate here.
"""

from __future__ import annotations

import numpy as np

DEFAULT_SEED = 20260803
AQ4_GROUP = 128
E4M3_MAX = 448.0

# ---------------------------------------------------------------------------
# scalar format helpers
# ---------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 bit patterns.

    NaN maps to the quiet NaN 0x7fc0 (sign kept); everything else follows the
    usual ``(bits + 0x7fff + lsb) >> 16`` rule.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    b = x.view(np.uint32).astype(np.uint64)
    lsb = (b >> 16) & 1
    r = ((b + 0x7FFF + lsb) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, ((b >> 16) & 0x8000 | 0x7FC0).astype(np.uint16), r)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 -> fp32 (values representable in bf16)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for code in range(256):
        s = -1.0 if code & 0x80 else 1.0
        e = (code >> 3) & 0xF
        m = code & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** -6
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[code] = v
    return t


E4M3_TABLE = _e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """e4m3fn code (uint8) -> fp32 value (exact)."""
    return E4M3_TABLE[np.ascontiguousarray(codes, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3fn code, round-to-nearest-even, saturating to +-448.

    Inputs are expected to be finite; NaN encodes to 0x7f.  Written as
    arithmetic on the value grid (not as a bit trick) so that it is independent
    of the device converter it checks.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.minimum(a, E4M3_MAX)
    # exponent of the grid cell: normal numbers use floor(log2 a) clamped to >= -6
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)  # spacing of representable values in this binade
    k = np.rint(a / step)  # ties-to-even on the integer grid; exact in fp64
    v = k * step  # may carry into the next binade: still representable
    v = np.minimum(v, E4M3_MAX)
    # encode the representable magnitude v
    with np.errstate(divide="ignore"):
        ev = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    normal = v >= 2.0 ** -6
    ev = np.clip(ev, -6, 8)
    mant = np.where(normal, np.rint((v / 2.0 ** ev - 1.0) * 8.0), np.rint(v / 2.0 ** -9))
    expf = np.where(normal, ev + 7, 0)
    code = (expf.astype(np.int64) << 3 | mant.astype(np.int64)).astype(np.uint8) | sign
    code = np.where(np.isnan(x), np.uint8(0x7F), code).astype(np.uint8)
    return code


# ---------------------------------------------------------------------------
# AQ4
# ---------------------------------------------------------------------------


def aq4_storage_bytes(elements: int, group: int = AQ4_GROUP, scale_bytes: int = 2) -> int:
    """Byte count of an AQ4 tensor in the style of Nvfp4 storage_bytes
    (crates/ullm-core/src/dtype.rs:100-122): ceil(n/2) + ceil(n/group)*scale."""
    return (elements + 1) // 2 + ((elements + group - 1) // group) * scale_bytes


def aq4_quantize(w: np.ndarray, group: int = AQ4_GROUP):
    """fp32 W[N,K] -> (packed uint8 [N,K/2], scales float16 [N,K/group])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    if k % group or group % 2:
        raise ValueError("K must be a multiple of the (even) group size")
    if not np.isfinite(w).all():
        raise ValueError("non-finite weights are outside the AQ4 contract")
    g = w.reshape(n, k // group, group)
    amax = np.abs(g).max(axis=2)
    s32 = (amax / np.float32(7.0)).astype(np.float32)
    s32 = np.minimum(s32, np.float32(65504.0))
    scales = s32.astype(np.float16)  # numpy casts with round-to-nearest-even
    sf = scales.astype(np.float32)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = (g / sf).astype(np.float32)  # single fp32 division, as on device
    q = np.where(sf == 0, np.float32(0), np.rint(ratio))
    q = np.clip(q, -7, 7).astype(np.int8).reshape(n, k)
    u = (q + 8).astype(np.uint8)
    packed = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
    return packed, scales


def aq4_unpack(packed: np.ndarray) -> np.ndarray:
    """packed uint8 [N,K/2] -> int8 q [N,K] in [-8,7] (codes 1..15 -> -7..7)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    n, kb = packed.shape
    q = np.empty((n, kb * 2), dtype=np.int8)
    q[:, 0::2] = (packed & 0xF).astype(np.int8) - 8
    q[:, 1::2] = (packed >> 4).astype(np.int8) - 8
    return q


def aq4_pack(q: np.ndarray) -> np.ndarray:
    """int8 q [N,K] in [-8,7] -> packed uint8 [N,K/2] (inverse of aq4_unpack)."""
    u = (np.ascontiguousarray(q, dtype=np.int8).astype(np.int16) + 8).astype(np.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def aq4_dequantize(packed: np.ndarray, scales: np.ndarray, group: int = AQ4_GROUP) -> np.ndarray:
    """-> fp32 W'[N,K]; q*scale is exact in fp32 (4-bit int times 11-bit significand)."""
    q = aq4_unpack(packed).astype(np.float32)
    n, k = q.shape
    sf = np.ascontiguousarray(scales, dtype=np.float16).astype(np.float32)
    return (q.reshape(n, k // group, group) * sf[:, :, None]).reshape(n, k).astype(np.float32)


# ---------------------------------------------------------------------------
# FP8 per-output-channel
# ---------------------------------------------------------------------------


def fp8_quantize(w: np.ndarray):
    """fp32 W[N,K] -> (codes uint8 [N,K], scale float32 [N])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if not np.isfinite(w).all():
        raise ValueError("non-finite weights are outside the FP8 contract")
    amax = np.abs(w).max(axis=1) if w.shape[1] else np.zeros(w.shape[0], np.float32)
    scale = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = (w / scale[:, None]).astype(np.float32)
    r = np.where(scale[:, None] == 0, np.float32(0), r)
    r = np.clip(r, -E4M3_MAX, E4M3_MAX).astype(np.float32)
    return e4m3_encode(r), scale


def fp8_dequantize(codes: np.ndarray, scale: np.ndarray) -> np.ndarray:
    return (e4m3_decode(codes) * np.ascontiguousarray(scale, np.float32)[:, None]).astype(np.float32)


# ---------------------------------------------------------------------------
# NVFP4
# ---------------------------------------------------------------------------

NVFP4_BLOCK = 16
_E2M1_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def e2m1_decode(codes: np.ndarray) -> np.ndarray:
    c = np.asarray(codes, np.uint8)
    return np.where(c & 8, -_E2M1_MAG[c & 7], _E2M1_MAG[c & 7]).astype(np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """Round to nearest on the e2m1 grid, ties to the even code, saturating at 6; returns 4-bit codes."""
    x = np.asarray(x, np.float32)
    a = np.minimum(np.abs(x), np.float32(6.0))
    # midpoints between neighbours; at a midpoint the even code (0, 2, 4, 6 -> 0, 1, 2, 4) wins
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    idx = np.zeros(a.shape, np.uint8)
    for i, m in enumerate(mids):
        up = (a > m) | ((a == m) & ((i + 1) % 2 == 0))  # crossing into code i+1: on a tie only if i+1 is even
        idx = np.where(up, np.uint8(i + 1), idx)
    sign = (np.signbit(x) & (idx != 0)).astype(np.uint8) << 3  # no negative zero codes
    return (idx | sign).astype(np.uint8)


def nvfp4_scale_bytes(n: int, k: int) -> int:
    return (n * (k // NVFP4_BLOCK) * 2 + 15) // 16 * 16 + 4


def nvfp4_quantize(w: np.ndarray):
    """fp32 [N,K] (K % 16 == 0) -> (packed u8 [N,K/2], block scales f16 [N,K/16], tensor scale f32 scalar)."""
    w = np.asarray(w, np.float32)
    n, k = w.shape
    assert k % NVFP4_BLOCK == 0
    amax_t = np.float32(np.abs(w).max()) if w.size else np.float32(0)
    if amax_t > 0:
        m, e = np.frexp(np.float32(amax_t / np.float32(6.0)))  # amax/6 = m * 2^e, m in [0.5, 1)
        ts = np.float32(np.ldexp(np.float32(1.0), int(e) - 1))
    else:
        ts = np.float32(1.0)
    blocks = w.reshape(n, k // NVFP4_BLOCK, NVFP4_BLOCK)
    amax_b = np.abs(blocks).max(axis=2)
    sb = ((amax_b / np.float32(6.0)).astype(np.float32) / ts).astype(np.float32).astype(np.float16)
    step = (sb.astype(np.float32) * ts).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = (blocks / step[:, :, None]).astype(np.float32)
    codes = np.where(step[:, :, None] > 0, e2m1_encode(np.nan_to_num(scaled, nan=0.0, posinf=6.0, neginf=-6.0)), np.uint8(0))
    codes = codes.reshape(n, k).astype(np.uint8)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, sb, ts


def nvfp4_dequantize(packed: np.ndarray, sb: np.ndarray, ts) -> np.ndarray:
    packed = np.asarray(packed, np.uint8)
    n, kb = packed.shape
    codes = np.empty((n, kb * 2), np.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    v = e2m1_decode(codes).reshape(n, kb * 2 // NVFP4_BLOCK, NVFP4_BLOCK)
    out = (v * np.asarray(sb, np.float16).astype(np.float32)[:, :, None]).astype(np.float32) * np.float32(ts)
    return out.astype(np.float32).reshape(n, kb * 2)


# ---------------------------------------------------------------------------
# linear, glue, error metric
# ---------------------------------------------------------------------------


def linear(x_bf16_as_f32: np.ndarray, w_deq: np.ndarray, out: str = "bf16") -> np.ndarray:
    """y = x @ w'^T with fp64 accumulation; ``out`` = 'bf16' (rounded, returned
    as fp32 values), 'f32' or 'f64'."""
    acc = x_bf16_as_f32.astype(np.float64) @ w_deq.astype(np.float64).T
    if out == "f64":
        return acc
    y = acc.astype(np.float32)
    return bf16_round(y) if out == "bf16" else y


def rmsnorm(x: np.ndarray, eps: float = 1e-5, gamma: np.ndarray | None = None) -> np.ndarray:
    """RMSNorm of bf16-valued rows with an optional bf16-valued weight vector gamma [K]:
    bf16( x * rsqrt(mean(x^2) + eps) * gamma ), fp64 inside, ONE rounding at the end."""
    x64 = x.astype(np.float64)
    r = 1.0 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + eps)
    y = x64 * r
    if gamma is not None:
        y = y * np.asarray(gamma, np.float64)[None, :]
    return bf16_round(y.astype(np.float32))


def swiglu(gate_up: np.ndarray) -> np.ndarray:
    """[M, 2F] (gate | up halves) -> bf16( silu(gate) * up ), fp64 inside."""
    f = gate_up.shape[1] // 2
    g = gate_up[:, :f].astype(np.float64)
    u = gate_up[:, f:].astype(np.float64)
    return bf16_round((g / (1.0 + np.exp(-g)) * u).astype(np.float32))


def error_stats(y: np.ndarray, ref: np.ndarray) -> dict:
    """Error report used by every parity test (all fields always present).

    pass := max_rel_floored <= 1e-2 and mean_abs <= 1e-3, where
    max_rel_floored = max |y-r| / max(|r|, 0.05*rms(r)) — element-wise relative
    error is ill-posed next to zero crossings, so the denominator is floored.
    """
    y = np.asarray(y, dtype=np.float64).ravel()
    r = np.asarray(ref, dtype=np.float64).ravel()
    bad = ~np.isfinite(y)
    d = np.abs(np.where(bad, 0.0, y) - r)
    rms = float(np.sqrt(np.mean(r * r))) if r.size else 0.0
    floor = max(0.05 * rms, 1e-30)
    stats = {
        "n": int(r.size),
        "max_abs": float(d.max()) if r.size else 0.0,
        "mean_abs": float(d.mean()) if r.size else 0.0,
        "max_rel_norm": float(d.max() / max(np.abs(r).max(), 1e-30)) if r.size else 0.0,
        "max_rel_floored": float((d / np.maximum(np.abs(r), floor)).max()) if r.size else 0.0,
        "outliers": int((d > 1e-3 + 1e-2 * np.abs(r)).sum()),
        "nan": int(np.isnan(y).sum()),
        "inf": int(np.isinf(y).sum()),
    }
    stats["pass"] = bool(
        stats["nan"] == 0 and stats["inf"] == 0 and stats["max_rel_floored"] <= 1e-2 and stats["mean_abs"] <= 1e-3
    )
    return stats


# ---------------------------------------------------------------------------
# counter-based synthetic generator (bit-identical in numpy, C and CUDA)
# ---------------------------------------------------------------------------

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def stream_key(seed: int, tensor_id: int) -> int:
    """64-bit key of one tensor's random stream."""
    k = _splitmix64(np.array([(seed & 0xFFFFFFFFFFFFFFFF)], dtype=np.uint64))[0]
    k = _splitmix64(np.array([k ^ np.uint64(tensor_id & 0xFFFFFFFFFFFFFFFF)], dtype=np.uint64))[0]
    return int(k)


def synth_normal(seed: int, tensor_id: int, start: int, count: int) -> np.ndarray:
    """Elements [start, start+count) of tensor ``tensor_id``: approximately
    N(0,1) as an Irwin-Hall sum of twelve 16-bit uniforms, computed in integers
    so that every implementation produces identical bits:
        z = float(2*S - 12*65535) * 2^-17,  S = sum of 12 uint16 draws.
    Draw j of element i is 16 bits of splitmix64(key + 3*i + j//4)."""
    key = np.uint64(stream_key(seed, tensor_id))
    idx = np.arange(start, start + count, dtype=np.uint64)
    s = np.zeros(count, dtype=np.int64)
    with np.errstate(over="ignore"):
        for j in range(3):
            h = _splitmix64((key + np.uint64(3) * idx + np.uint64(j)) & _M64)
            for p in range(4):
                s += ((h >> np.uint64(16 * p)) & np.uint64(0xFFFF)).astype(np.int64)
    return ((2 * s - 12 * 65535).astype(np.float32) * np.float32(2.0 ** -17)).astype(np.float32)


def synth_weights(seed: int, tensor_id: int, n: int, k: int, row0: int = 0, std: float = 0.02) -> np.ndarray:
    """Rows [row0,row0+n) of a [*,K] fp32 weight tensor: fp32(std) * z."""
    z = synth_normal(seed, tensor_id, row0 * k, n * k)
    return (z * np.float32(std)).astype(np.float32).reshape(n, k)


def synth_activations(seed: int, tensor_id: int, m: int, k: int) -> np.ndarray:
    """bf16_rne(z) as fp32 values, shape [M,K]."""
    return bf16_round(synth_normal(seed, tensor_id, 0, m * k)).reshape(m, k)


def planted_case_weights(seed: int, tensor_id: int, n: int, k: int) -> np.ndarray:
    """Synthetic weights with the format's edge cases planted in rows 0-2 (n >= 3,
    k >= 128): an all-zero group, a lone outlier, and a group whose scale is
    exactly 1.0 holding +-x.5 ties (round-half-even: 0.5->0, 1.5->2, 2.5->2, 6.5->6)."""
    w = synth_weights(seed, tensor_id, n, k)
    w[0, :128] = 0.0
    w[1, 5] = 1.0
    w[2, :128] = 0.0
    w[2, 0] = 7.0
    w[2, 1:8] = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 6.5, -6.5], np.float32)
    return w


# ---------------------------------------------------------------------------
# linear stack (tiny shapes only: every weight is materialised in fp32)
# ---------------------------------------------------------------------------

STACK_QKV, STACK_O, STACK_GATE_UP, STACK_DOWN, STACK_LM_HEAD = 0, 1, 2, 3, 4


def stack_tensor_id(layer: int, which: int) -> int:
    """Random-stream id of one full (unsharded) stack weight."""
    return (layer << 8) | which | (1 << 40)


def stack_norm_tensor_id(layer: int, which: int) -> int:
    """Random-stream id of the RMSNorm weight vector in front of one column-parallel stack linear."""
    return (layer << 8) | which | (2 << 40)


def stack_gamma(seed, layer, which, k) -> np.ndarray:
    """gamma[i] = bf16(1 + z_i / 8) as fp32 values, z the counter-based normal stream."""
    z = synth_normal(seed, stack_norm_tensor_id(layer, which), 0, k)
    return bf16_round((np.float32(1.0) + z * np.float32(0.125)).astype(np.float32))


def stack_weight(seed, layer, which, n, k, encoding: str):
    """Dequantised full weight [n,k] of one stack linear ('aq4' or 'fp8')."""
    w = synth_weights(seed, stack_tensor_id(layer, which), n, k)
    if encoding == "aq4":
        return aq4_dequantize(*aq4_quantize(w))
    return fp8_dequantize(*fp8_quantize(w))


def stack_reference(seed, encoding, layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab, x, eps=1e-5,
                    trace=None):
    """One pass of the linear stack on bf16-valued x [m, hidden] -> logits (bf16
    values) [m, vocab].  The residual stream h is fp32.  Dataflow per layer:
        qkv = QKV(rmsnorm(bf16(h), g1));  h = h + O(qkv[:, :q_dim])        (fp32 add)
        act = swiglu(GateUp(rmsnorm(bf16(h), g2)));  h = h + Down(act)
    then logits = LMHead(rmsnorm(bf16(h), gf)).  `trace`, if a dict, receives every
    intermediate under (layer, which) (for O and Down: the new h)."""
    qd, kvd = q_heads * head_dim, kv_heads * head_dim
    h = x.astype(np.float32)
    for l in range(layers):
        g1, g2 = stack_gamma(seed, l, STACK_QKV, hidden), stack_gamma(seed, l, STACK_GATE_UP, hidden)
        qkv = linear(rmsnorm(bf16_round(h), eps, g1), stack_weight(seed, l, STACK_QKV, qd + 2 * kvd, hidden, encoding))
        h1 = (h + linear(qkv[:, :qd], stack_weight(seed, l, STACK_O, hidden, qd, encoding), out="f32")).astype(np.float32)
        gu = swiglu(linear(rmsnorm(bf16_round(h1), eps, g2), stack_weight(seed, l, STACK_GATE_UP, 2 * ffn, hidden, encoding)))
        h = (h1 + linear(gu, stack_weight(seed, l, STACK_DOWN, hidden, ffn, encoding), out="f32")).astype(np.float32)
        if trace is not None:
            trace[(l, STACK_QKV)], trace[(l, STACK_O)] = qkv, h1
            trace[(l, STACK_GATE_UP)], trace[(l, STACK_DOWN)] = gu, h
    gf = stack_gamma(seed, 0, STACK_LM_HEAD, hidden)
    return linear(rmsnorm(bf16_round(h), eps, gf), stack_weight(seed, 0, STACK_LM_HEAD, vocab, hidden, encoding))

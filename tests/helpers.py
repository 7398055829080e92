"""Helpers shared by the GPU parity tests: device-side tensors built through the
C ABI, and the oracle-side reference for one linear."""
import numpy as np

import oracle as o
import ullm_cuda as U
from ullm_cuda import _abi as abi

SEED = o.DEFAULT_SEED
CANARY = 0xC5


class DeviceWeight:
    """A quantised weight living in device buffers, built from fp32 host data by
    the CUDA quantiser (so the test also covers quantise -> consume)."""

    def __init__(self, ctx, q, w_f32: np.ndarray, encoding: int):
        n, k = w_f32.shape
        self.n, self.k, self.encoding = n, k, encoding
        vb, sb = U.weight_bytes(encoding, n, k)
        self.vb, self.sb = vb, sb
        self.src = ctx.alloc(max(w_f32.nbytes, 16))
        self.values = ctx.alloc(vb + 256)  # 256 canary bytes after the payload
        self.scales = ctx.alloc(sb + 256)
        q.fill(self.values.at(0), CANARY, vb + 256)
        q.fill(self.scales.at(0), CANARY, sb + 256)
        q.upload(self.src.at(0), w_f32)
        self.desc = U.weight_desc(encoding, n, k, self.values.at(0), self.scales.at(0))
        q.quantize(self.src.at(0), self.desc)

    def download(self, q):
        if self.encoding == U.ENCODING_AQ4:
            v = q.download(self.values.at(0), (self.n, self.k // 2), np.uint8)
            s = q.download(self.scales.at(0), (self.n, self.k // 128), np.float16)
        else:
            v = q.download(self.values.at(0), (self.n, self.k), np.uint8)
            s = q.download(self.scales.at(0), (self.n,), np.float32)
        return v, s

    def canaries_intact(self, q) -> bool:
        a = q.download(self.values.at(self.vb), (256,), np.uint8)
        b = q.download(self.scales.at(self.sb), (256,), np.uint8)
        return bool((a == CANARY).all() and (b == CANARY).all())

    def close(self):
        for b in (self.src, self.values, self.scales):
            b.close()


def oracle_quantize(w, encoding):
    return o.aq4_quantize(w) if encoding == U.ENCODING_AQ4 else o.fp8_quantize(w)


def oracle_dequantize(v, s, encoding):
    return o.aq4_dequantize(v, s) if encoding == U.ENCODING_AQ4 else o.fp8_dequantize(v, s)


def run_linear(ctx, q, dw: DeviceWeight, x_vals: np.ndarray, *, x_dtype=U.DTYPE_BF16, y_dtype=U.DTYPE_BF16,
               prologue=U.PROLOGUE_NONE, kernel=U.KERNEL_AUTO, x_stride=0, y_stride=0, submit=True,
               epilogue=U.EPILOGUE_NONE, gamma=None, residual=None):
    """x_vals: fp32 array [M, cols] (bf16-representable unless x_dtype is F32); gamma: bf16-valued fp32 [K] or
    None; residual: fp32 [M, N] or None.  Returns (y as fp32 values [M, N], completion result or None)."""
    m, cols = x_vals.shape
    xs = x_stride or cols
    n_out = dw.n // 2 if epilogue == U.EPILOGUE_SWIGLU else dw.n
    ys = y_stride or n_out
    xe = 2 if x_dtype == U.DTYPE_BF16 else 4
    ye = 2 if y_dtype == U.DTYPE_BF16 else 4
    xbuf = ctx.alloc(m * xs * xe + 256)
    ybuf = ctx.alloc(m * ys * ye + 256)
    host = np.zeros((m, xs), np.float32)
    host[:, :cols] = x_vals
    q.upload(xbuf.at(0), o.f32_to_bf16_bits(host).reshape(m, xs) if x_dtype == U.DTYPE_BF16 else host)
    q.fill(ybuf.at(0), CANARY, m * ys * ye + 256)
    extra = []
    gt = rt = None
    if gamma is not None:
        gbuf = ctx.alloc(len(gamma) * 2)
        q.upload(gbuf.at(0), o.f32_to_bf16_bits(np.asarray(gamma, np.float32)))
        gt = gbuf.at(0)
        extra.append(gbuf)
    if residual is not None:
        rbuf = ctx.alloc(residual.size * 4)
        q.upload(rbuf.at(0), np.ascontiguousarray(residual, np.float32))
        rt = rbuf.at(0)
        extra.append(rbuf)
    d = U.linear_desc(dw.desc, m, xbuf.at(0), ybuf.at(0), input_dtype=x_dtype, output_dtype=y_dtype,
                      prologue=prologue, kernel=kernel, input_row_stride=x_stride, output_row_stride=y_stride,
                      epilogue=epilogue, norm_weight=gt, residual=rt)
    res = None
    if submit:
        res = q.linear_submit(d).wait(60000)
    else:
        q.linear_enqueue(d)
        q.synchronize()
    raw = q.download(ybuf.at(0), (m * ys * ye + 256,), np.uint8)
    assert (raw[m * ys * ye:] == CANARY).all(), "kernel wrote past the output span"
    body = raw[: m * ys * ye]
    if y_dtype == U.DTYPE_BF16:
        y = o.bf16_bits_to_f32(body.view(np.uint16)).reshape(m, ys)
    else:
        y = body.view(np.float32).reshape(m, ys)
    if ys > n_out:  # padding columns of a strided output must be untouched
        pad = raw[: m * ys * ye].reshape(m, ys * ye)[:, n_out * ye:]
        assert (pad == CANARY).all(), "kernel wrote into the row padding"
    for b in [xbuf, ybuf] + extra:
        b.close()
    return y[:, :n_out].copy(), res


def oracle_linear(x_vals, w_deq, prologue=U.PROLOGUE_NONE, x_is_f32=False, out="bf16", eps=1e-5,
                  epilogue=U.EPILOGUE_NONE, gamma=None, residual=None):
    x = o.bf16_round(x_vals.astype(np.float32)) if x_is_f32 else x_vals
    if prologue == U.PROLOGUE_RMSNORM:
        x = o.rmsnorm(x, eps, gamma)
    elif prologue == U.PROLOGUE_SWIGLU:
        x = o.swiglu(x)
    if epilogue == U.EPILOGUE_SWIGLU:  # rows [gate | up] -> bf16(silu(bf16 gate) * bf16 up)
        return o.swiglu(o.linear(x, w_deq, out="bf16"))
    if residual is None:
        return o.linear(x, w_deq, out=out)
    y = (o.linear(x, w_deq, out="f64") + residual.astype(np.float64)).astype(np.float32)  # added before the output rounding
    return o.bf16_round(y) if out == "bf16" else y

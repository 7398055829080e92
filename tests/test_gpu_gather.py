"""The fused all-reduce of the tensor-parallel decode path, checked on ONE GPU through its two single-op halves:
every "rank" is a slot of one device buffer, filled by one launch after the other (row-parallel shards of the
same linear), then gathered by the linear that follows — the very kernels the multi-GPU stack launches, with 2, 4
and 8 ranks' slot layouts, gathered once per thread block and once per thread-block cluster.  Also the failure
path in its sanctioned form: a slot that nobody fills makes the wait run out after a short limit, the kernel
returns, and the host reports DEVICE_FLAGGED (no fault, no hang)."""
import time

import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, DeviceWeight, oracle_dequantize, oracle_linear, oracle_quantize

pytestmark = pytest.mark.gpu
ENCODINGS = [U.ENCODING_AQ4, U.ENCODING_FP8_CHANNEL]


def _fill_slots(ctx, q, enc, ranks, m, hidden, k_full, seed_off, slots, stride, tag, skip=()):
    """Row-parallel linear hidden <- k_full cut into `ranks` K shards; returns the fp64 sum of the partials."""
    w = o.synth_weights(SEED, 3000 + seed_off, hidden, k_full)
    x = o.synth_activations(SEED, 3100 + seed_off, m, k_full)
    ks = k_full // ranks
    total = np.zeros((m, hidden), np.float64)
    xb = ctx.alloc(m * ks * 2)
    dummy = ctx.alloc(m * hidden * 4)
    for r in range(ranks):
        wr = np.ascontiguousarray(w[:, r * ks:(r + 1) * ks])
        dw = DeviceWeight(ctx, q, wr, enc)  # each shard quantised on its own, on the device and in the oracle
        wdq = oracle_dequantize(*oracle_quantize(wr, enc), enc)
        xr = np.ascontiguousarray(x[:, r * ks:(r + 1) * ks])
        total += o.linear(xr, wdq, out="f64")
        if r not in skip:
            q.upload(xb.at(0), o.f32_to_bf16_bits(xr).reshape(m, ks))
            q.linear_enqueue_partial(U.linear_desc(dw.desc, m, xb.at(0), dummy.at(0), output_dtype=U.DTYPE_F32),
                                     U.slots_desc(slots.at(0), stride, ranks, rank=r, tag=tag))
            q.synchronize()
        dw.close()
    xb.close()
    dummy.close()
    return total


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("ranks,m,gather", [(2, 1, 0), (2, 3, 1), (4, 1, 1), (4, 2, 0), (8, 1, 0), (8, 1, 1), (8, 4, 1)])
def test_partial_then_reduced_matches_the_oracle(gpu, encoding, ranks, m, gather):
    ctx, q = gpu
    hidden, k_full, n2 = 1024, 2048, 640
    stride = m * hidden * 8 + 256
    slots = ctx.alloc(ranks * stride)
    q.fill(slots.at(0), 0, ranks * stride)
    resid = (o.synth_normal(SEED, 3200 + m, 0, m * hidden).reshape(m, hidden)).astype(np.float32)
    gamma = o.bf16_round((1.0 + 0.125 * o.synth_normal(SEED, 3300, 0, hidden)).astype(np.float32))
    w2 = o.synth_weights(SEED, 3400 + ranks, n2, hidden)
    dw2 = DeviceWeight(ctx, q, w2, encoding)
    w2dq = oracle_dequantize(*oracle_quantize(w2, encoding), encoding)
    rb, gb = ctx.alloc(resid.nbytes), ctx.alloc(hidden * 2)
    q.upload(rb.at(0), resid)
    q.upload(gb.at(0), o.f32_to_bf16_bits(gamma))
    red, yb, xdummy = ctx.alloc(m * hidden * 4), ctx.alloc(m * n2 * 2), ctx.alloc(m * hidden * 4)
    for tag in (7, 8):  # two uses of the same slots: the tag tells fresh values from stale ones
        total = _fill_slots(ctx, q, encoding, ranks, m, hidden, k_full, tag, slots, stride, tag)
        d = U.linear_desc(dw2.desc, m, xdummy.at(0), yb.at(0), input_dtype=U.DTYPE_F32, prologue=U.PROLOGUE_RMSNORM,
                          norm_weight=gb.at(0), residual=rb.at(0))
        q.linear_enqueue_reduced(d, U.slots_desc(slots.at(0), stride, ranks, tag=tag, gather=gather), red.at(0))
        r = q.synchronize()
        assert r.device_flags == 0
        h = q.download(red.at(0), (m, hidden), np.float32)
        h_ref = (resid.astype(np.float64) + total).astype(np.float32)
        st = o.error_stats(h, h_ref)
        assert st["max_rel_floored"] <= 1e-4 and st["nan"] == 0, st  # fp32 sums of fp32 partials
        y = o.bf16_bits_to_f32(q.download(yb.at(0), (m, n2), np.uint16))
        ref = oracle_linear(h, w2dq, U.PROLOGUE_RMSNORM, x_is_f32=True, gamma=gamma)  # on the device's own sum
        st = o.error_stats(y, ref)
        assert st["pass"], (ranks, m, gather, st)
    for b in (slots, rb, gb, red, yb, xdummy):
        b.close()
    dw2.close()


@pytest.mark.parametrize("gather", [0, 1])
def test_a_wait_that_runs_out_returns_and_is_reported(gather):
    """One of two slots is never filled.  With a 50 ms limit the gathering kernel gives up, the work queued behind
    it returns without waiting again, the completion reports device_flags and DEVICE_FLAGGED, and the context
    serves the next op normally.  The wait gives up and returns: nothing faults and nothing hangs."""
    ctx = U.Context(0)
    ctx.set_wait_limit(50)
    q = ctx.queue()
    enc, ranks, m, hidden, n2 = U.ENCODING_FP8_CHANNEL, 2, 1, 1024, 256
    stride = m * hidden * 8
    slots = ctx.alloc(ranks * stride)
    q.fill(slots.at(0), 0, ranks * stride)
    _fill_slots(ctx, q, enc, ranks, m, hidden, 2048, 1, slots, stride, 5, skip=(1,))
    w2 = o.synth_weights(SEED, 3500, n2, hidden)
    dw2 = DeviceWeight(ctx, q, w2, enc)
    yb, xdummy = ctx.alloc(m * n2 * 2), ctx.alloc(m * hidden * 4)
    d = U.linear_desc(dw2.desc, m, xdummy.at(0), yb.at(0), input_dtype=U.DTYPE_F32)
    t0 = time.perf_counter()
    for _ in range(4):  # four gathers in a row: only the first may spend the limit
        q.linear_enqueue_reduced(d, U.slots_desc(slots.at(0), stride, ranks, tag=5, gather=gather))
    c = q.signal()
    with pytest.raises(U.CudaError) as e:
        c.wait(30000)
    elapsed = time.perf_counter() - t0
    assert e.value.status is U.Status.DeviceFlagged, e.value
    assert c.last_result.device_flags != 0
    assert elapsed < 5.0, f"the queue took {elapsed:.2f} s to unwind four gathers with a 50 ms limit"
    # the flag and the abort word are re-armed: an ordinary linear and a complete gather work again
    x = o.synth_activations(SEED, 3600, m, hidden)
    xb = ctx.alloc(m * hidden * 2)
    q.upload(xb.at(0), o.f32_to_bf16_bits(x).reshape(m, hidden))
    r = q.linear_submit(U.linear_desc(dw2.desc, m, xb.at(0), yb.at(0))).wait(30000)
    assert r.device_flags == 0
    y = o.bf16_bits_to_f32(q.download(yb.at(0), (m, n2), np.uint16))
    assert o.error_stats(y, oracle_linear(x, oracle_dequantize(*oracle_quantize(w2, enc), enc)))["pass"]
    _fill_slots(ctx, q, enc, ranks, m, hidden, 2048, 1, slots, stride, 6)
    q.linear_enqueue_reduced(d, U.slots_desc(slots.at(0), stride, ranks, tag=6, gather=gather))
    assert q.synchronize().device_flags == 0
    for b in (slots, yb, xdummy, xb):
        b.close()
    dw2.close()
    q.close()
    ctx.close()


def test_slots_argument_errors(gpu):
    ctx, q = gpu
    w = o.synth_weights(SEED, 3700, 128, 256)
    dw = DeviceWeight(ctx, q, w, U.ENCODING_FP8_CHANNEL)
    xb, yb, sl = ctx.alloc(256 * 4), ctx.alloc(128 * 4), ctx.alloc(4096)
    d = U.linear_desc(dw.desc, 1, xb.at(0), yb.at(0), output_dtype=U.DTYPE_F32)
    for kw, status in ((dict(ranks=9), U.Status.InvalidArgument), (dict(ranks=2, rank=2), U.Status.InvalidArgument),
                       (dict(ranks=2, stride=1000), U.Status.InvalidArgument),  # not a multiple of 16
                       (dict(ranks=8, stride=1024), U.Status.OutOfRange)):      # leaves the 4096-byte buffer
        with pytest.raises(U.CudaError) as e:
            q.linear_enqueue_partial(d, U.slots_desc(sl.at(0), kw.get("stride", 1024), kw["ranks"], rank=kw.get("rank", 0)))
        assert e.value.status is status, (kw, e.value)
    with pytest.raises(U.CudaError) as e:  # the gather is offered for the plain and RMSNorm prologues only
        q.linear_enqueue_reduced(U.linear_desc(dw.desc, 1, xb.at(0), yb.at(0), prologue=U.PROLOGUE_SWIGLU),
                                 U.slots_desc(sl.at(0), 2048, 2))
    assert e.value.status in (U.Status.Unsupported, U.Status.OutOfRange)
    for b in (xb, yb, sl):
        b.close()
    dw.close()

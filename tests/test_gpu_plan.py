"""The coarse command-list boundary on a GPU: prepare (metadata copied, kernels chosen) -> submit (bindings with
access modes, dependency events across queues) -> event query / wait -> shutdown with drain.  Shapes follow the
projections of one decoder block; results are checked against the oracle per op (each op on the device's own input).
Reference anchors: docs/architecture/runtime.md:53-63, :77-79; crates/ullm-core/src/handles.rs:12-16, :100-145."""
import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from ullm_cuda import _abi as abi
from helpers import SEED, DeviceWeight, oracle_dequantize, oracle_linear, oracle_quantize

pytestmark = pytest.mark.gpu
R, W, RW = abi.ACCESS_READ, abi.ACCESS_WRITE, abi.ACCESS_READ_WRITE


def _block(ctx, q, enc, m, hidden, ffn):
    """Weights, buffers and bindings of: h2 = h + O(x) (residual in place), act = swiglu(GateUp(rmsnorm(h2, g)))."""
    wo = o.synth_weights(SEED, 5000, hidden, hidden)
    wg = o.synth_weights(SEED, 5001, 2 * ffn, hidden)
    dwo, dwg = DeviceWeight(ctx, q, wo, enc), DeviceWeight(ctx, q, wg, enc)
    x = o.synth_activations(SEED, 5002, m, hidden)
    h = o.synth_normal(SEED, 5003, 0, m * hidden).reshape(m, hidden).astype(np.float32)
    g = o.bf16_round((1.0 + 0.125 * o.synth_normal(SEED, 5004, 0, hidden)).astype(np.float32))
    xb, hb, gb, ab = ctx.alloc(m * hidden * 2), ctx.alloc(m * hidden * 4), ctx.alloc(hidden * 2), ctx.alloc(m * ffn * 2)
    q.upload(xb.at(0), o.f32_to_bf16_bits(x).reshape(m, hidden))
    q.upload(hb.at(0), h)
    q.upload(gb.at(0), o.f32_to_bf16_bits(g))
    ops = [U.plan_op(enc, m, hidden, hidden, output_dtype=U.DTYPE_F32, residual=True),
           U.plan_op(enc, m, 2 * ffn, hidden, input_dtype=U.DTYPE_F32, prologue=U.PROLOGUE_RMSNORM, epilogue=U.EPILOGUE_SWIGLU,
                     norm_weight=True)]
    bindings = [U.binding(0, abi.SLOT_WEIGHT_VALUES, R, dwo.desc.values), U.binding(0, abi.SLOT_WEIGHT_SCALES, R, dwo.desc.scales),
                U.binding(0, abi.SLOT_INPUT, R, xb.at(0)), U.binding(0, abi.SLOT_OUTPUT, RW, hb.at(0)),
                U.binding(0, abi.SLOT_RESIDUAL, R, hb.at(0)),
                U.binding(1, abi.SLOT_WEIGHT_VALUES, R, dwg.desc.values), U.binding(1, abi.SLOT_WEIGHT_SCALES, R, dwg.desc.scales),
                U.binding(1, abi.SLOT_INPUT, R, hb.at(0)), U.binding(1, abi.SLOT_OUTPUT, W, ab.at(0)),
                U.binding(1, abi.SLOT_NORM_WEIGHT, R, gb.at(0))]
    wodq = oracle_dequantize(*oracle_quantize(wo, enc), enc)
    wgdq = oracle_dequantize(*oracle_quantize(wg, enc), enc)
    refs = dict(x=x, h=h, g=g, wodq=wodq, wgdq=wgdq)
    return ops, bindings, (dwo, dwg, xb, hb, gb, ab), refs


@pytest.mark.parametrize("encoding", [U.ENCODING_AQ4, U.ENCODING_FP8_CHANNEL])
@pytest.mark.parametrize("m", [1, 24])
def test_prepare_submit_wait_matches_the_oracle(gpu, encoding, m):
    ctx, q = gpu
    hidden, ffn = 512, 384
    ops, bindings, bufs, r = _block(ctx, q, encoding, m, hidden, ffn)
    plan = U.Prepared(ctx, ops)
    ops[0].n = 7  # prepare copied the metadata: the caller's array may change or go away
    ev = plan.submit(q, bindings)
    ev.wait(60000)
    assert ev.query() == abi.EVENT_SUCCESS and ev.query() == abi.EVENT_SUCCESS  # not consumed
    hb, ab = bufs[3], bufs[5]
    h2 = q.download(hb.at(0), (m, hidden), np.float32)
    st = o.error_stats(h2, oracle_linear(r["x"], r["wodq"], out="f32", residual=r["h"]))
    assert st["pass"], st
    act = o.bf16_bits_to_f32(q.download(ab.at(0), (m, ffn), np.uint16))
    ref = oracle_linear(h2, r["wgdq"], U.PROLOGUE_RMSNORM, x_is_f32=True, epilogue=U.EPILOGUE_SWIGLU, gamma=r["g"])
    st = o.error_stats(act, ref)
    assert st["nan"] == 0 and st["mean_abs"] <= 1e-3 and st["outliers"] <= max(2, act.size // 2000), st
    ev.close()
    plan.close()
    for b in bufs:
        b.close()


def test_dependency_events_order_two_queues(gpu):
    """Submission B on another queue waits for A's event: B's input is A's output."""
    ctx, q1 = gpu
    q2 = ctx.queue()
    enc, m, k, n = U.ENCODING_FP8_CHANNEL, 4, 2048, 2048
    w1, w2 = o.synth_weights(SEED, 5100, n, k), o.synth_weights(SEED, 5101, 256, n)
    d1, d2 = DeviceWeight(ctx, q1, w1, enc), DeviceWeight(ctx, q1, w2, enc)
    x = o.synth_activations(SEED, 5102, m, k)
    xb, mid, yb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2), ctx.alloc(m * 256 * 2)
    q1.upload(xb.at(0), o.f32_to_bf16_bits(x).reshape(m, k))
    q1.fill(mid.at(0), 0, m * n * 2)
    q1.synchronize()
    pa = U.Prepared(ctx, [U.plan_op(enc, m, n, k)] * 1)
    pb = U.Prepared(ctx, [U.plan_op(enc, m, 256, n)])
    ba = [U.binding(0, abi.SLOT_WEIGHT_VALUES, R, d1.desc.values), U.binding(0, abi.SLOT_WEIGHT_SCALES, R, d1.desc.scales),
          U.binding(0, abi.SLOT_INPUT, R, xb.at(0)), U.binding(0, abi.SLOT_OUTPUT, W, mid.at(0))]
    bb = [U.binding(0, abi.SLOT_WEIGHT_VALUES, R, d2.desc.values), U.binding(0, abi.SLOT_WEIGHT_SCALES, R, d2.desc.scales),
          U.binding(0, abi.SLOT_INPUT, R, mid.at(0)), U.binding(0, abi.SLOT_OUTPUT, W, yb.at(0))]
    for _ in range(5):
        ea = pa.submit(q1, ba)
        eb = pb.submit(q2, bb, wait=[ea])
        eb.wait(60000)
        assert ea.query() == abi.EVENT_SUCCESS  # B ran after A
        ea.close()
        eb.close()
    midv = o.bf16_bits_to_f32(q1.download(mid.at(0), (m, n), np.uint16))
    y = o.bf16_bits_to_f32(q2.download(yb.at(0), (m, 256), np.uint16))
    assert o.error_stats(midv, oracle_linear(x, oracle_dequantize(*oracle_quantize(w1, enc), enc)))["pass"]
    assert o.error_stats(y, oracle_linear(midv, oracle_dequantize(*oracle_quantize(w2, enc), enc)))["pass"]
    for h in (pa, pb, d1, d2, xb, mid, yb, q2):
        h.close()


def test_submit_validates_bindings_and_access_modes(gpu):
    ctx, q = gpu
    ops, bindings, bufs, _ = _block(ctx, q, U.ENCODING_FP8_CHANNEL, 2, 256, 128)
    plan = U.Prepared(ctx, ops)

    def rejected(bs, status=U.Status.InvalidArgument):
        with pytest.raises(U.CudaError) as e:
            plan.submit(q, bs)
        assert e.value.status is status, e.value

    rejected(bindings[:-1])                                     # op 1's norm weight is not bound
    rejected(bindings + [bindings[2]])                          # a slot bound twice
    ro = list(bindings)
    ro[3] = U.binding(0, abi.SLOT_OUTPUT, R, bufs[3].at(0))     # output bound read-only
    rejected(ro)
    wo = list(bindings)
    wo[2] = U.binding(0, abi.SLOT_INPUT, W, bufs[2].at(0))      # input bound write-only
    rejected(wo)
    alias = list(bindings)
    alias[3] = U.binding(0, abi.SLOT_OUTPUT, W, bufs[3].at(0))  # output == residual needs READ_WRITE
    rejected(alias)
    clash = list(bindings)
    clash[8] = U.binding(1, abi.SLOT_OUTPUT, W, bufs[3].at(0))  # op 1 would write what it reads
    rejected(clash)
    rejected(bindings + [U.binding(0, abi.SLOT_NORM_WEIGHT, R, bufs[4].at(0))])  # op 0 was prepared without a norm weight
    rejected(bindings + [U.binding(5, abi.SLOT_INPUT, R, bufs[2].at(0))])        # no such op
    small = list(bindings)
    small[8] = U.binding(1, abi.SLOT_OUTPUT, W, bufs[5].at(16 * 1024 * 1024))    # span leaves its buffer
    rejected(small, U.Status.OutOfRange)
    with pytest.raises(U.CudaError) as e:  # a plan is validated at prepare time: no kernel serves a ragged K
        U.Prepared(ctx, [U.plan_op(U.ENCODING_AQ4, 1, 256, 200)])
    assert e.value.status is U.Status.Unsupported
    plan.submit(q, bindings).wait(60000)  # and the untouched bindings are fine
    plan.close()
    for b in bufs:
        b.close()


def test_a_failure_after_enqueue_lives_in_the_event_and_shutdown_drains():
    """A device-side wait that gives up (a gather on a slot nobody fills, 50 ms limit) is not a submit failure:
    submit returns OK, the event turns to FAILURE with its own diagnostic, shutdown counts it, refuses new work, and
    the executor kept watching a submission whose event the caller had dropped."""
    ctx = U.Context(0)
    ctx.set_wait_limit(50)
    q = ctx.queue()
    enc, hidden = U.ENCODING_FP8_CHANNEL, 1024
    dw = DeviceWeight(ctx, q, o.synth_weights(SEED, 5200, 256, hidden), enc)
    xb, yb, slots = ctx.alloc(hidden * 4), ctx.alloc(256 * 2), ctx.alloc(2 * hidden * 8)
    q.fill(slots.at(0), 0, 2 * hidden * 8)
    q.fill(xb.at(0), 0, hidden * 4)
    q.synchronize()
    plan = U.Prepared(ctx, [U.plan_op(enc, 1, 256, hidden, input_dtype=U.DTYPE_F32)])
    bs = [U.binding(0, abi.SLOT_WEIGHT_VALUES, R, dw.desc.values), U.binding(0, abi.SLOT_WEIGHT_SCALES, R, dw.desc.scales),
          U.binding(0, abi.SLOT_INPUT, R, xb.at(0)), U.binding(0, abi.SLOT_OUTPUT, W, yb.at(0))]
    # the gather that will give up runs in front of the plan on the same queue
    q.linear_enqueue_reduced(U.linear_desc(dw.desc, 1, xb.at(0), yb.at(0), input_dtype=U.DTYPE_F32),
                             U.slots_desc(slots.at(0), hidden * 8, 2, tag=4))
    ev = plan.submit(q, bs)                      # OK: nothing is wrong with the submission itself
    dropped = plan.submit(q, bs, want_event=False)
    assert dropped is None
    with pytest.raises(U.CudaError) as e:
        ev.wait(30000)
    assert e.value.status is U.Status.DeviceFlagged and "bounded wait" in e.value.message
    with pytest.raises(U.CudaError) as e2:      # the event owns its diagnostic: the same answer again
        ev.query()
    assert e2.value.status is U.Status.DeviceFlagged
    failed = ctx.shutdown(30000)
    assert failed >= 0                           # (the failure was already collected by the wait above)
    with pytest.raises(U.CudaError) as e3:
        plan.submit(q, bs)
    assert e3.value.status is U.Status.InvalidArgument and "shutting down" in e3.value.message
    with pytest.raises(U.CudaError):
        U.Prepared(ctx, [U.plan_op(enc, 1, 256, hidden)])
    for h in (ev, plan, dw, xb, yb, slots, q):
        h.close()
    ctx.close()

"""Lifecycle rules of the boundary on a GPU: destructors never block on the device, a completion is consumed by
every outcome of wait (a timeout included), queues of one context do not share GEMM staging memory, and one process
may drive several devices (function attributes are set per device)."""
import time

import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, DeviceWeight, oracle_dequantize, oracle_linear, oracle_quantize

pytestmark = pytest.mark.gpu


def _gemm_case(ctx, q, m, n, k, enc, seed_off):
    w = o.synth_weights(SEED, 4000 + seed_off, n, k)
    dw = DeviceWeight(ctx, q, w, enc)
    x = o.synth_activations(SEED, 4100 + seed_off, m, k)
    xb, yb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
    q.upload(xb.at(0), o.f32_to_bf16_bits(x).reshape(m, k))
    ref = oracle_linear(x, oracle_dequantize(*oracle_quantize(w, enc), enc))
    return dw, xb, yb, ref


def test_wait_consumes_the_completion_on_timeout_too():
    """native/hip/src/hip_evidence_runtime.hip.cpp:691-716: every outcome of wait retires the handle."""
    ctx = U.Context(0)
    ctx.set_wait_limit(300)
    q = ctx.queue()
    # something that takes a while without faulting: a gather whose second slot is never filled gives up after 300 ms
    hidden = 1024
    slots = ctx.alloc(2 * hidden * 8)
    q.fill(slots.at(0), 0, 2 * hidden * 8)
    dw = DeviceWeight(ctx, q, o.synth_weights(SEED, 4200, 128, hidden), U.ENCODING_FP8_CHANNEL)
    xd, yb = ctx.alloc(hidden * 4), ctx.alloc(128 * 2)
    d = U.linear_desc(dw.desc, 1, xd.at(0), yb.at(0), input_dtype=U.DTYPE_F32)
    q.linear_enqueue_reduced(d, U.slots_desc(slots.at(0), hidden * 8, 2, tag=3))
    c = q.signal()
    handle = c.handle.value
    with pytest.raises(U.CudaError) as e:
        c.wait(1)  # 1 ms: the kernel is still waiting for its peer
    assert e.value.status is U.Status.Timeout
    lib = U.abi.load()
    import ctypes as C
    assert lib.ullm_cuda_completion_wait(C.c_void_p(handle), 0, None, None) == U.abi.CUDA_INVALID_HANDLE
    assert lib.ullm_cuda_completion_query(C.c_void_p(handle), 0, None) == U.abi.CUDA_INVALID_HANDLE
    # destroying the queue while that kernel still runs returns at once; the context can only go once the
    # queue's background retirement has finished
    t0 = time.perf_counter()
    q.close()
    assert time.perf_counter() - t0 < 0.1
    deadline = time.time() + 20
    while True:
        try:
            for b in (slots, xd, yb):
                if b.handle.value:
                    b.close()
            dw.close()
            ctx.close()
            break
        except U.CudaError as err:
            assert err.status is U.Status.InvalidArgument and time.time() < deadline, err
            time.sleep(0.05)


def test_gemm_linears_on_two_queues_of_one_context_do_not_share_staging():
    ctx = U.Context(0)
    q1, q2 = ctx.queue(), ctx.queue()
    a = _gemm_case(ctx, q1, 300, 512, 1024, U.ENCODING_FP8_CHANNEL, 1)
    b = _gemm_case(ctx, q2, 200, 384, 2048, U.ENCODING_AQ4, 2)
    for _ in range(20):  # interleaved: the two streams overlap on the GPU
        q1.linear_enqueue(U.linear_desc(a[0].desc, 300, a[1].at(0), a[2].at(0), kernel=U.KERNEL_GEMM))
        q2.linear_enqueue(U.linear_desc(b[0].desc, 200, b[1].at(0), b[2].at(0), kernel=U.KERNEL_GEMM))
    assert q1.synchronize().device_flags == 0 and q2.synchronize().device_flags == 0
    ya = o.bf16_bits_to_f32(q1.download(a[2].at(0), (300, 512), np.uint16))
    yb = o.bf16_bits_to_f32(q2.download(b[2].at(0), (200, 384), np.uint16))
    assert o.error_stats(ya, a[3])["pass"] and o.error_stats(yb, b[3])["pass"]
    for dw, xb, yb_, _ in (a, b):
        dw.close()
        xb.close()
        yb_.close()
    q1.close()
    q2.close()
    ctx.close()


def test_one_process_two_devices():
    """Contexts on device 0 and 1 in one process, a 256-token GEMM and a large-K matvec on each: the kernels'
    shared-memory attributes are raised per device."""
    if U.backend_probe().device_count < 2:
        pytest.skip("needs two GPUs")
    for dev in (0, 1):
        ctx = U.Context(dev)
        q = ctx.queue()
        for enc in (U.ENCODING_FP8_CHANNEL, U.ENCODING_AQ4):
            dw, xb, yb, ref = _gemm_case(ctx, q, 256, 256, 1024, enc, 10 + dev)
            q.linear_submit(U.linear_desc(dw.desc, 256, xb.at(0), yb.at(0), kernel=U.KERNEL_GEMM)).wait(60000)
            assert o.error_stats(o.bf16_bits_to_f32(q.download(yb.at(0), (256, 256), np.uint16)), ref)["pass"], (dev, enc)
            for h in (dw, xb, yb):
                h.close()
            dw, xb, yb, ref = _gemm_case(ctx, q, 1, 300, 14336, enc, 20 + dev)
            q.linear_submit(U.linear_desc(dw.desc, 1, xb.at(0), yb.at(0), kernel=U.KERNEL_MATVEC)).wait(60000)
            assert o.error_stats(o.bf16_bits_to_f32(q.download(yb.at(0), (1, 300), np.uint16)), ref)["pass"], (dev, enc)
            for h in (dw, xb, yb):
                h.close()
        q.close()
        ctx.close()

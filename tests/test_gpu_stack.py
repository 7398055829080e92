"""GPU parity of the decoder linear stack (one rank) against the NumPy chain, plus
full-size spot checks that re-derive one linear from the stack's own buffers."""
import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from helpers import SEED, oracle_dequantize, oracle_linear, oracle_quantize

pytestmark = pytest.mark.gpu

TINY = U.StackShape(layers=3, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1000)


def _read(q, span, shape, dtype_id):
    if dtype_id == U.DTYPE_F32:
        return q.download(span, shape, np.float32)
    return o.bf16_bits_to_f32(q.download(span, shape, np.uint16))


@pytest.mark.parametrize("encoding,name", [(U.ENCODING_AQ4, "aq4"), (U.ENCODING_FP8_CHANNEL, "fp8")])
@pytest.mark.parametrize("m", [1, 5, 8])
@pytest.mark.parametrize("flags", [0, U.STACK_FLAG_NO_GRAPH])
def test_tiny_stack_every_linear_matches_the_oracle(gpu, encoding, name, m, flags):
    """Every one of the 13 linears is checked at the stated tolerance against the oracle
    applied to the DEVICE's own input of that linear.  (A chain of bf16 roundings is
    chaotic at the 1-ulp level — one flipped rounding upstream flips a few percent of
    the roundings downstream — so the end-to-end logits are only held to a loose bound.)"""
    ctx, q = gpu
    st = U.Stack(ctx, q, TINY, encoding, max_tokens=8, flags=flags | U.STACK_FLAG_KEEP_ACTIVATIONS)
    x = o.synth_activations(SEED, 900 + m, m, TINY.hidden)
    xb = o.f32_to_bf16_bits(x).reshape(m, TINY.hidden)
    y = None
    for _ in range(2):  # second pass replays the captured graph
        y = o.bf16_bits_to_f32(st.step_host(xb))
    qd = TINY.q_heads * TINY.head_dim
    linears = [(l, w) for l in range(TINY.layers) for w in (U.LINEAR_QKV, U.LINEAR_O, U.LINEAR_GATE_UP, U.LINEAR_DOWN)]
    linears.append((0, U.LINEAR_LM_HEAD))
    for layer, which in linears:
        info = st.linear_info(layer, which)
        n, k = int(info.weight.n), int(info.weight.k)
        in_cols = {U.LINEAR_O: qd + 2 * TINY.kv_heads * TINY.head_dim}.get(which, k)
        xin = _read(q, info.last_input, (m, in_cols), info.input_dtype)
        if which == U.LINEAR_O:
            xin = xin[:, :qd]  # the O projection reads the query part of the fused QKV output
        n_out = n // 2 if info.epilogue == U.EPILOGUE_SWIGLU else n
        yout = _read(q, info.last_output, (m, n_out), info.output_dtype)
        wdq = o.stack_weight(SEED, layer, which, n, k, name)
        gamma = resid = None
        if info.norm_weight.buffer:  # the RMSNorm weight vector is the seeded one
            gamma = o.bf16_bits_to_f32(q.download(info.norm_weight, (k,), np.uint16))
            assert np.array_equal(gamma, o.stack_gamma(SEED, layer, which, k)), (layer, which)
            assert info.norm_tensor_id == o.stack_norm_tensor_id(layer, which)
        if info.last_residual.buffer:  # row-parallel linears: the residual stream they added their result to
            resid = q.download(info.last_residual, (m, n), np.float32)
        assert bool(info.norm_weight.buffer) == (which in (U.LINEAR_QKV, U.LINEAR_GATE_UP, U.LINEAR_LM_HEAD))
        assert bool(info.last_residual.buffer) == (which in (U.LINEAR_O, U.LINEAR_DOWN))
        ref = oracle_linear(xin, wdq, info.prologue, x_is_f32=info.input_dtype == U.DTYPE_F32,
                            out="f32" if info.output_dtype == U.DTYPE_F32 else "bf16", epilogue=info.epilogue,
                            gamma=gamma, residual=resid)
        stt = o.error_stats(yout, ref)
        if info.epilogue == U.EPILOGUE_SWIGLU:
            # the epilogue works on bf16 gate|up values: a gate that sits on a rounding tie flips by one ulp with
            # the accumulation order, and silu's slope amplifies that beyond 1e-2 of a small output
            assert stt["nan"] == 0 and stt["mean_abs"] <= 1e-3 and stt["outliers"] <= max(2, yout.size // 2000), (layer, which, stt)
        else:
            assert stt["pass"], (layer, which, stt)
    ref = o.stack_reference(SEED, name, TINY.layers, TINY.hidden, TINY.q_heads, TINY.kv_heads, TINY.head_dim,
                            TINY.ffn, TINY.vocab, x)
    assert np.sqrt(np.mean((y - ref) ** 2)) < 0.02 * np.sqrt(np.mean(ref ** 2))
    # device-resident entry gives the same bits as the host entry
    xin, yout = ctx.alloc(xb.nbytes), ctx.alloc(m * TINY.vocab * 2)
    q.upload(xin.at(0), xb)
    st.step(m, xin.at(0), yout.at(0))
    q.synchronize()
    assert np.array_equal(q.download(yout.at(0), (m, TINY.vocab), np.uint16), st.step_host(xb))
    wb, launches = st.stats()
    linears = TINY.layers * 4 + 1  # one matvec launch each, or activation planes + GEMM (+ SwiGLU) on the tensor-core path
    assert linears + 1 <= launches <= 3 * linears + 1  # + the kernel that starts the residual stream
    per = {U.ENCODING_AQ4: lambda n, k: n * k // 2 + n * k // 64, U.ENCODING_FP8_CHANNEL: lambda n, k: n * k + 4 * n}[encoding]
    want = TINY.layers * (per(qd + 2 * TINY.kv_heads * TINY.head_dim, TINY.hidden) + per(TINY.hidden, qd)
                          + per(2 * TINY.ffn, TINY.hidden) + per(TINY.hidden, TINY.ffn)) + per(TINY.vocab, TINY.hidden)
    assert wb == want
    xin.close()
    yout.close()
    st.close()


def test_stack_weights_are_the_seeded_quantised_tensors(gpu):
    ctx, q = gpu
    st = U.Stack(ctx, q, TINY, U.ENCODING_FP8_CHANNEL, max_tokens=2)
    for layer, which, n, k in ((1, U.LINEAR_O, 256, 256), (2, U.LINEAR_DOWN, 256, 512), (0, U.LINEAR_LM_HEAD, 1000, 256)):
        info = st.linear_info(layer, which)
        assert (info.weight.n, info.weight.k, info.full_n, info.full_k) == (n, k, n, k)
        w = o.synth_weights(SEED, info.tensor_id, n, k)
        v, s = o.fp8_quantize(w)
        assert np.array_equal(q.download(info.weight.values, (n, k), np.uint8), v)
        assert np.array_equal(q.download(info.weight.scales, (n,), np.float32), s)
        assert info.tensor_id == o.stack_tensor_id(layer if which != U.LINEAR_LM_HEAD else 0, which)
    st.close()


def test_stack_argument_errors(gpu):
    ctx, q = gpu
    with pytest.raises(U.CudaError) as e:
        U.Stack(ctx, q, U.StackShape(1, 200, 4, 2, 50, 512, 1000), U.ENCODING_AQ4, max_tokens=1)  # K not /128
    assert e.value.status is U.Status.Unsupported
    with pytest.raises(U.CudaError) as e:
        U.Stack(ctx, q, TINY, U.ENCODING_AQ4, max_tokens=1, tp_size=2, tp_rank=0)  # no comm
    assert e.value.status is U.Status.InvalidHandle
    st = U.Stack(ctx, q, TINY, U.ENCODING_AQ4, max_tokens=2)
    with pytest.raises(U.CudaError) as e:
        st.step_host(np.zeros((3, TINY.hidden), np.uint16))
    assert e.value.status is U.Status.InvalidArgument
    st.close()


def test_one_full_width_layer_spot_check(gpu):
    """A 1-layer stack at Llama-3-8B widths: the last linear's device input and
    output are read back and a strided sample of its rows is recomputed by the oracle."""
    ctx, q = gpu
    shape = U.StackShape(1, 4096, 32, 8, 128, 14336, 4096)  # vocab cut to keep the test light
    for encoding in (U.ENCODING_AQ4, U.ENCODING_FP8_CHANNEL):
        st = U.Stack(ctx, q, shape, encoding, max_tokens=2)
        x = o.synth_activations(SEED, 950, 2, shape.hidden)
        st.step_host(o.f32_to_bf16_bits(x).reshape(2, shape.hidden))
        for which, k_in_cols in ((U.LINEAR_DOWN, 14336), (U.LINEAR_GATE_UP, 4096)):
            info = st.linear_info(0, which)
            n, k = int(info.weight.n), int(info.weight.k)
            pair = info.epilogue == U.EPILOGUE_SWIGLU
            in_dt = np.float32 if info.input_dtype == U.DTYPE_F32 else np.uint16
            xin = q.download(info.last_input, (2, k_in_cols), in_dt)
            xin = xin if in_dt == np.float32 else o.bf16_bits_to_f32(xin)
            out_dt = np.float32 if info.output_dtype == U.DTYPE_F32 else np.uint16
            yout = q.download(info.last_output, (2, n // 2 if pair else n), out_dt)
            yout = yout if out_dt == np.float32 else o.bf16_bits_to_f32(yout)
            cols = np.arange(0, n // 2 if pair else n, 331)
            rows = np.concatenate([cols, n // 2 + cols]) if pair else cols  # gate rows, then the matching up rows
            wr = np.stack([o.synth_weights(SEED, info.tensor_id, 1, k, row0=int(r))[0] for r in rows])
            v, s = oracle_quantize(wr, encoding)
            gamma = o.bf16_bits_to_f32(q.download(info.norm_weight, (k,), np.uint16)) if info.norm_weight.buffer else None
            resid = q.download(info.last_residual, (2, n), np.float32)[:, cols] if info.last_residual.buffer else None
            ref = oracle_linear(xin, oracle_dequantize(v, s, encoding), info.prologue, x_is_f32=in_dt == np.float32,
                                out="f32" if out_dt == np.float32 else "bf16", epilogue=info.epilogue, gamma=gamma,
                                residual=resid)
            stt = o.error_stats(yout[:, cols], ref)
            assert stt["pass"], (encoding, which, stt)
        st.close()

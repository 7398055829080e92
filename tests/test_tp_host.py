"""CPU tests of the tensor-parallel host logic with gloo ranks (world size 2): the shard plan
(which rows / columns of each full weight a rank owns) reassembles to the unsharded linear,
and the NCCL-id exchange the bench uses works over torch.distributed.  No GPU is involved;
the device all-reduce itself is exercised on multi-GPU runs of the bench."""
import os
import subprocess
import sys
import textwrap

import numpy as np

import oracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def shard_plan(hidden, q_heads, kv_heads, head_dim, ffn, vocab, tp, rank):
    """Mirror of the stack's sharding rule: column-parallel QKV (by head), gate+up (gate and up rows
    split alike) and LM head; row-parallel O and down (contiguous K slices)."""
    qd, kvd = q_heads * head_dim, kv_heads * head_dim
    ql, kvl, fl, vl = qd // tp, kvd // tp, ffn // tp, vocab // tp
    return {
        "qkv_rows": np.concatenate([np.arange(rank * ql, (rank + 1) * ql), qd + np.arange(rank * kvl, (rank + 1) * kvl),
                                    qd + kvd + np.arange(rank * kvl, (rank + 1) * kvl)]),
        "o_cols": np.arange(rank * ql, (rank + 1) * ql),
        "gate_up_rows": np.concatenate([np.arange(rank * fl, (rank + 1) * fl), ffn + np.arange(rank * fl, (rank + 1) * fl)]),
        "down_cols": np.arange(rank * fl, (rank + 1) * fl),
        "lm_rows": np.arange(rank * vl, (rank + 1) * vl),
    }


def test_shards_reassemble_to_the_unsharded_layer():
    hidden, qh, kvh, hd, ffn, vocab, tp = 256, 4, 2, 64, 512, 1000, 2
    seed, m = o.DEFAULT_SEED, 3
    x = o.synth_activations(seed, 1, m, hidden)
    wq = o.stack_weight(seed, 0, o.STACK_QKV, (qh + 2 * kvh) * hd, hidden, "fp8")
    wo = o.stack_weight(seed, 0, o.STACK_O, hidden, qh * hd, "fp8")
    wgu = o.stack_weight(seed, 0, o.STACK_GATE_UP, 2 * ffn, hidden, "aq4")
    wd = o.stack_weight(seed, 0, o.STACK_DOWN, hidden, ffn, "aq4")
    qkv_full = o.linear(x, wq)
    o_full = o.linear(qkv_full[:, : qh * hd], wo, out="f32")
    act_full = o.swiglu(o.linear(x, wgu))
    d_full = o.linear(act_full, wd, out="f32")
    o_sum = np.zeros_like(o_full)
    d_sum = np.zeros_like(d_full)
    covered = []
    for rank in range(tp):
        pl = shard_plan(hidden, qh, kvh, hd, ffn, vocab, tp, rank)
        qkv_local = o.linear(x, wq[pl["qkv_rows"]])
        ql = qh * hd // tp
        assert np.array_equal(qkv_local[:, :ql], qkv_full[:, pl["o_cols"]])  # local query part = its slice
        o_sum += o.linear(qkv_local[:, :ql], wo[:, pl["o_cols"]], out="f32")
        act_local = o.swiglu(o.linear(x, wgu[pl["gate_up_rows"]]))  # [gate_l | up_l] rows keep the pairing local
        assert np.array_equal(act_local, act_full[:, pl["down_cols"]])
        d_sum += o.linear(act_local, wd[:, pl["down_cols"]], out="f32")
        covered.append(pl["lm_rows"])
    assert np.allclose(o_sum, o_full, rtol=1e-5, atol=1e-6)  # sum over ranks = the row-parallel all-reduce
    assert np.allclose(d_sum, d_full, rtol=1e-5, atol=1e-6)
    assert np.array_equal(np.concatenate(covered), np.arange(vocab))
    # AQ4 groups of 128 never straddle a row-parallel split at the benchmark shapes
    for k, t in ((4096, 8), (14336, 8), (8192, 8), (28672, 8)):
        assert (k // t) % 128 == 0


def test_fp8_row_parallel_shards_use_full_row_scales():
    """A K-slice of a row quantised over the FULL row keeps the full row's codes: every TP degree computes
    with the same quantised weights."""
    w = o.synth_weights(o.DEFAULT_SEED, 77, 8, 512)
    codes, scale = o.fp8_quantize(w)
    part_codes, part_scale = o.fp8_quantize(w[:, :256])
    assert not np.array_equal(part_scale, scale) or np.array_equal(part_codes, codes[:, :256])
    assert np.array_equal(o.fp8_dequantize(codes, scale)[:, 256:], o.fp8_dequantize(codes[:, 256:], scale))


def test_two_gloo_ranks_exchange_an_id_and_reduce_timings(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent("""
        import os, sys
        import torch, torch.distributed as dist
        dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
        rank = dist.get_rank()
        box = [bytes(range(128)) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)           # how the bench ships the NCCL unique id
        assert box[0] == bytes(range(128))
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)         # max over ranks of a timing
        assert t.item() == 2.0
        dist.barrier()
        dist.destroy_process_group()
        print("ok", rank)
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29571", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("ok" in out for out in outs)

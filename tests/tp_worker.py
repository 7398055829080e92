"""One tensor-parallel rank of the multi-GPU stack test (launched by tests/test_gpu_tp.py, one
process per GPU).  Builds a small stack at tp_size = WORLD_SIZE, runs one step, and checks this
rank's slice of the logits against the NumPy chain; rank 0 also checks a tp_size = 1 stack on
its own GPU against the same reference."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "ullm-project_b200"), os.path.join(ROOT, "oracle")):
    sys.path.insert(0, p)

import torch.distributed as dist  # noqa: E402

import oracle as o  # noqa: E402
import ullm_cuda as U  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    enc_name = sys.argv[1]
    m = int(sys.argv[2])
    enc = U.ENCODING_AQ4 if enc_name == "aq4" else U.ENCODING_FP8_CHANNEL
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = U.Context(rank)
    q = ctx.queue()
    box = [U.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = U.Comm(ctx, box[0], rank, world)
    # every per-rank K stays a multiple of 128 up to eight ranks (q 1024 / 8, ffn 1024 / 8), eight KV heads
    shape = U.StackShape(layers=2, hidden=512, q_heads=16, kv_heads=8, head_dim=64, ffn=1024, vocab=2048)
    seed = o.DEFAULT_SEED
    x = o.synth_activations(seed, 990 + m, m, shape.hidden)
    xb = o.f32_to_bf16_bits(x).reshape(m, shape.hidden)
    ref = o.stack_reference(seed, enc_name, shape.layers, shape.hidden, shape.q_heads, shape.kv_heads, shape.head_dim,
                            shape.ffn, shape.vocab, x)
    mode = sys.argv[3] if len(sys.argv) > 3 else "push"
    nccl_only = mode == "nccl"
    flags = {"nccl": U.STACK_FLAG_NCCL_ONLY, "push": 0, "push-block": U.STACK_FLAG_GATHER_PER_BLOCK,
             "push-cluster": U.STACK_FLAG_GATHER_PER_CLUSTER}[mode]
    st = U.Stack(ctx, q, shape, enc, max_tokens=m, tp_rank=rank, tp_size=world, comm=comm,
                 flags=U.STACK_FLAG_KEEP_ACTIVATIONS | flags)
    y = None
    for _ in range(2):
        y = o.bf16_bits_to_f32(st.step_host(xb))
    vl = shape.vocab // world
    mine = ref[:, rank * vl:(rank + 1) * vl]
    # a chain of bf16 roundings is only reproducible to the 1-ulp level end to end (see the stack test)
    err = float(np.sqrt(np.mean((y - mine) ** 2)) / np.sqrt(np.mean(mine ** 2)))
    assert err < 0.02, err
    _, launches = st.stats()
    # one kernel per linear on the matvec path (the sum over ranks fused into them, plus the step tick), up to
    # three on the tensor-core path (activation planes, GEMM, SwiGLU), plus one ncclAllReduce after O and after
    # down when the sum is not fused
    linears = shape.layers * 4 + 1
    assert linears + 1 <= launches <= 1 + 3 * linears + 2 * shape.layers, launches
    if m == 1 and not nccl_only:
        assert launches in (linears + 1, linears + 1 + 2 * shape.layers), launches
    # EVERY row-parallel sum (O and down of every layer) at the stated tolerance: the device's own input of the
    # linear is gathered over the ranks' K shards, the full-K oracle linear plus the residual is the reference
    qd = shape.q_heads * shape.head_dim
    for layer in range(shape.layers):
        for which, full_k, in_cols in ((U.LINEAR_O, qd, (qd + 2 * shape.kv_heads * shape.head_dim) // world),
                                       (U.LINEAR_DOWN, shape.ffn, shape.ffn // world)):
            info = st.linear_info(layer, which)
            kl = full_k // world
            mine_in = o.bf16_bits_to_f32(q.download(info.last_input, (m, in_cols), np.uint16))[:, :kl]
            parts = [None] * world
            dist.all_gather_object(parts, np.ascontiguousarray(mine_in))
            x_full = np.concatenate(parts, axis=1)
            resid = q.download(info.last_residual, (m, shape.hidden), np.float32)
            got = q.download(info.last_output, (m, shape.hidden), np.float32)
            w_full = o.stack_weight(seed, layer, which, shape.hidden, full_k, enc_name)
            want = (o.linear(x_full, w_full, out="f64") + resid.astype(np.float64)).astype(np.float32)
            stt = o.error_stats(got, want)
            assert stt["max_rel_floored"] <= 1e-2 and stt["mean_abs"] <= 1e-3 and stt["nan"] == 0, (layer, which, stt)
    st.close()
    if rank == 0:
        st1 = U.Stack(ctx, q, shape, enc, max_tokens=m)
        y1 = o.bf16_bits_to_f32(st1.step_host(xb))
        e1 = float(np.sqrt(np.mean((y1 - ref) ** 2)) / np.sqrt(np.mean(ref ** 2)))
        assert e1 < 0.02, e1
        st1.close()
    dist.barrier()
    comm.close()
    q.close()
    ctx.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok err={err:.2e}")


if __name__ == "__main__":
    main()

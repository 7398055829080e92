"""Benchmark of the quantised-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--workload NAME] [--impl reference]

Default workload: one decode step of the Llama-3-70B-shaped FP8 (e4m3, per-channel
scale) linear stack, tensor-parallel over N GPUs of one node (column-parallel QKV /
gate+up / LM head, row-parallel O / down followed by an NCCL all-reduce), random-init
weights generated on the device from a seed, bf16 activations ~ N(0,1).  A "step" is
one pass of all 321 linears for a batch of B tokens; `value` is tokens/s of the whole
job with inputs resident in HBM; `e2e` is the same step driven through the host entry
point (pinned host input -> H2D -> step -> D2H of the logits).  The roofline object is
the decode matvec kernel: algorithmic bytes of a step's matvec launches over their
device time, against the measured HBM copy bandwidth.  No model checkpoint or dataset
is involved: the shapes are the only thing taken from the named model.

One process per GPU: for N > 1 launch with
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 ... bench.py --gpus N
(torch.distributed over gloo carries only the NCCL id, barriers and the max-over-ranks
reduction of the timings; all device work goes through libullm_cuda).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "ullm-project_b200"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

SEED = 20260803
WORKLOADS = {
    # name: (shape attr, encoding name, description)
    "stack70b-fp8": ("LLAMA3_70B", "fp8", "Llama-3-70B-shaped FP8 e4m3 linear stack, one decode step"),
    "stack8b-aq4": ("LLAMA3_8B", "aq4", "Llama-3-8B-shaped AQ4 linear stack, one decode step"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def stack_algorithmic_bytes(shape, enc, batch, tp):
    """Per rank and per step: packed weights + scales + activations read and written by the linears."""
    qd, kvd = shape.q_heads * shape.head_dim, shape.kv_heads * shape.head_dim
    per = (lambda n, k: n * k // 2 + n * k // 64) if enc == "aq4" else (lambda n, k: n * k + 4 * n)
    # (N, K, input bytes per element, output columns, output bytes per element)
    lin = [((qd + 2 * kvd) // tp, shape.hidden, 2, (qd + 2 * kvd) // tp, 2), (shape.hidden, qd // tp, 2, shape.hidden, 4),
           (2 * shape.ffn // tp, shape.hidden, 4, shape.ffn // tp, 2), (shape.hidden, shape.ffn // tp, 2, shape.hidden, 4)]
    w = shape.layers * sum(per(n, k) for n, k, _, _, _ in lin) + per(shape.vocab // tp, shape.hidden)
    a = shape.layers * sum(batch * (k * xi + cols * yo) for n, k, xi, cols, yo in lin)
    a += batch * (shape.hidden * 4 + shape.vocab // tp * 2)
    return w, a


def cpu_sample(shape, enc, batch, seconds_hint=15.0):
    """Times the plain-C port on ONE decoder layer (QKV, O, gate+up, down) of the same widths
    with all host threads and scales to the whole stack by weight elements."""
    import oracle_c as oc

    rng = np.random.default_rng(SEED)
    qd, kvd = shape.q_heads * shape.head_dim, shape.kv_heads * shape.head_dim
    lin = [(qd + 2 * kvd, shape.hidden), (shape.hidden, qd), (2 * shape.ffn, shape.hidden), (shape.hidden, shape.ffn)]
    mats = []
    for n, k in lin:
        x = oc.synth_activations_bits(SEED, 5000 + k, batch, k)
        if enc == "aq4":
            mats.append((x, rng.integers(0x11, 0xFF, (n, k // 2), dtype=np.uint8),
                         np.full((n, k // 128), 0.003, np.float16)))
        else:
            codes = rng.integers(0, 0x7E, (n, k), dtype=np.uint8) | (rng.integers(0, 2, (n, k), dtype=np.uint8) << 7)
            mats.append((x, codes, np.full(n, 1e-4, np.float32)))
    elems = sum(n * k for n, k in lin)

    def one_pass():
        t0 = time.perf_counter()
        for x, v, s in mats:
            (oc.linear_aq4 if enc == "aq4" else oc.linear_fp8)(x, v, s)
        return time.perf_counter() - t0

    return one_pass, elems, oc.num_threads()


def run_reference(args, shape, enc):
    """The reference project has no CPU (or any) implementation of this path, so the
    reference arm times this repository's plain-C port of the format spec on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    one_pass, elems, threads = cpu_sample(shape, enc, args.batch)
    reps = max(1, int(np.ceil(1.0 / max(one_pass(), 1e-4))))  # a step = about one second of host work
    for _ in range(args.warmup):
        one_pass()
    times = [sum(one_pass() for _ in range(reps)) / reps for _ in range(args.steps)]
    t = sum(times) / len(times)
    scale = shape.weight_elements() / elems
    value = args.batch / (t * scale)
    sample = (f"one decoder layer (QKV, O, gate+up, down; {elems} weight elements) of the same widths, {reps} passes "
              f"per step ({t * reps:.2f} s), scaled x{scale:.2f} to the whole stack by weight elements")
    line = {
        "impl": "reference", "metric": "linear-stack decode tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * scale * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[args.workload][2] + f", batch {args.batch}", "batch": args.batch,
                   "encoding": enc, "note": "CPU port of the spec (the reference has no implementation of this path)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_matvec_extra(U, ctx, q, enc_id, n, k, m, reps, kernel=None):
    """Time per launch of one matvec shape over enough distinct weight copies to exceed 2x L2,
    replayed as one graph (so the figure is HBM, not L2, and launch gaps are the graph's)."""
    vb, sb = U.weight_bytes(enc_id, n, k)
    copies = max(2, int(2 * 130e6 // (vb + sb)) + 1)
    src = ctx.alloc(n * k * 4)
    q.synth_weights(SEED, 4242, 0, n * k, 0.02, src.at(0))
    bufs, descs = [], []
    xb, yb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
    q.synth_activations(SEED, 4243, 0, m * k, xb.at(0))
    for _ in range(copies):
        v, s = ctx.alloc(vb), ctx.alloc(sb)
        wd = U.weight_desc(enc_id, n, k, v.at(0), s.at(0))
        q.quantize(src.at(0), wd)
        bufs += [v, s]
        descs.append(U.linear_desc(wd, m, xb.at(0), yb.at(0), kernel=U.KERNEL_MATVEC if kernel is None else kernel))
    q.linear_enqueue(descs[0])  # any scratch the kernel needs exists before the capture
    q.synchronize()
    q.capture_begin()
    for d in descs:
        q.linear_enqueue(d)
    g = q.capture_end()
    for _ in range(3):
        g.launch(q)
    q.synchronize()
    a = q.signal()
    for _ in range(reps):
        g.launch(q)
    b = q.signal()
    b.query(600000)
    ms = b.elapsed_ms_since(a)
    a.close()
    b.close()
    g.close()
    for buf in bufs + [src, xb, yb]:
        buf.close()
    us = ms * 1e3 / (reps * copies)
    algo = vb + sb + m * k * 2 + m * n * 2
    return {"us_per_launch": us, "algorithmic_bytes": algo, "gbs": algo / us / 1e3, "weight_copies": copies}


def tensor_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured (MEASURED_PEAKS.json)"
    return 1590.0, 1400.0, "fallback (1.59 PFLOP/s burst, earlier measurement on this pool)"


def time_gemm(U, ctx, q, enc_id, m, n, k, reps):
    """Device time of one fused-dequant GEMM launch (tcgen05 path), activations [m,k] bf16 resident in HBM."""
    vb, sb = U.weight_bytes(enc_id, n, k)
    src = ctx.alloc(n * k * 4)
    q.synth_weights(SEED, 4300, 0, n * k, 0.02, src.at(0))
    v, s = ctx.alloc(vb), ctx.alloc(sb)
    wd = U.weight_desc(enc_id, n, k, v.at(0), s.at(0))
    q.quantize(src.at(0), wd)
    src.close()
    xb, yb = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
    q.synth_activations(SEED, 4301, 0, m * k, xb.at(0))
    d = U.linear_desc(wd, m, xb.at(0), yb.at(0), kernel=U.KERNEL_GEMM)
    for _ in range(3):
        q.linear_enqueue(d)
    q.synchronize()
    a = q.signal()
    for _ in range(reps):
        q.linear_enqueue(d)
    b = q.signal()
    b.query(600000)
    ms = b.elapsed_ms_since(a) / reps
    a.close()
    b.close()
    for buf in (v, s, xb, yb):
        buf.close()
    flops = 2.0 * m * n * k
    return {"us_per_launch": ms * 1e3, "tflops": flops / (ms * 1e-3) / 1e12, "flops": flops,
            "weight_gbs": (vb + sb) / (ms * 1e-3) / 1e9}


def run_single_gemm(U, args):
    """One GEMM shape on one GPU: M = --batch tokens, weight [--n, --k]; prints TFLOP/s against the
    measured cuBLAS bf16 peak (burst: the kernel is timed alone)."""
    ctx = U.Context(0)
    q = ctx.queue()
    enc_id = U.ENCODING_AQ4 if args.enc == "aq4" else U.ENCODING_FP8_CHANNEL
    r = time_gemm(U, ctx, q, enc_id, args.batch, args.n, args.k, reps=max(args.steps, 1))
    burst, sustained, src = tensor_peaks()
    print(json.dumps({
        "metric": "fused-dequant GEMM TFLOP/s", "value": r["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": 3, "ms_per_step": r["us_per_launch"] / 1e3, "higher_is_better": True,
        "config": {"workload": f"{args.enc} GEMM M={args.batch} N={args.n} K={args.k}"},
        "roofline": {"bound": "tensor", "achieved": r["tflops"], "peak": burst, "unit": "TFLOP/s",
                     "frac": r["tflops"] / burst, "traffic": None, "peak_source": src,
                     "frac_of_sustained": r["tflops"] / sustained, "frac_of_nominal_2250": r["tflops"] / 2250.0,
                     "weight_stream_gbs": r["weight_gbs"]},
        "gpu_launches": max(args.steps, 1) + 3}), flush=True)
    q.close()
    ctx.close()


def run_single_matvec(U, args):
    """One matvec shape on one GPU (the case the ncu captures use): `--steps` graph replays over
    weight copies that together exceed 2x L2; prints achieved HBM GB/s against the measured peak."""
    ctx = U.Context(0)
    q = ctx.queue()
    enc_id = U.ENCODING_AQ4 if args.enc == "aq4" else U.ENCODING_FP8_CHANNEL
    kernel = {"auto": U.KERNEL_AUTO, "matvec": U.KERNEL_MATVEC, "gemm": U.KERNEL_GEMM}[args.kernel]
    r = time_matvec_extra(U, ctx, q, enc_id, args.n, args.k, args.batch, reps=max(args.steps, 1), kernel=kernel)
    peak, peak_src = peaks()
    print(json.dumps({
        "metric": "quantised matvec HBM GB/s", "value": r["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": 3, "ms_per_step": r["us_per_launch"] * r["weight_copies"] / 1e3, "higher_is_better": True,
        "config": {"workload": f"{args.enc} matvec M={args.batch} N={args.n} K={args.k}", "weight_copies": r["weight_copies"],
                   "kernel": args.kernel},
        "roofline": {"bound": "hbm", "achieved": r["gbs"], "peak": peak, "unit": "GB/s", "frac": r["gbs"] / peak,
                     "traffic": None, "peak_source": peak_src, "us_per_launch": r["us_per_launch"],
                     "algorithmic_bytes": r["algorithmic_bytes"]},
        "gpu_launches": r["weight_copies"] * (max(args.steps, 1) + 3)}), flush=True)
    q.close()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--workload", default="stack70b-fp8", choices=sorted(WORKLOADS) + ["matvec", "gemm"])
    ap.add_argument("--enc", default="fp8", choices=["fp8", "aq4"], help="matvec workload: weight encoding")
    ap.add_argument("--kernel", default="auto", choices=["auto", "matvec", "gemm"],
                    help="matvec workload: kernel behind the linear op (auto: by token count)")
    ap.add_argument("--n", type=int, default=57344, help="matvec workload: output channels")
    ap.add_argument("--k", type=int, default=8192, help="matvec workload: reduction length")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; the line says so)")
    ap.add_argument("--no-extra", action="store_true", help="skip the single-matvec figures and the CPU baseline")
    ap.add_argument("--nccl-only", action="store_true", help="sum over ranks with ncclAllReduce instead of the fused peer-memory push")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    import ullm_cuda as U

    if args.workload == "matvec":
        run_single_matvec(U, args)
        return
    if args.workload == "gemm":
        run_single_gemm(U, args)
        return
    shape_name, enc, descr = WORKLOADS[args.workload]
    shape = getattr(U, shape_name)
    if args.layers:
        shape = U.StackShape(args.layers, shape.hidden, shape.q_heads, shape.kv_heads, shape.head_dim, shape.ffn, shape.vocab)
    if args.impl == "reference":
        run_reference(args, shape, enc)
        return
    enc_id = U.ENCODING_AQ4 if enc == "aq4" else U.ENCODING_FP8_CHANNEL

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch one process per GPU with torch.distributed.run")
    dist = None
    if world > 1:
        import torch.distributed as dist  # plumbing only: NCCL id, barrier, max over ranks
        dist.init_process_group("gloo", rank=rank, world_size=world)

    probe = U.backend_probe()
    if not probe.available:
        raise SystemExit(f"no usable B200: {probe.diagnostic} (there is no CPU fallback to measure)")
    ctx = U.Context(local)
    q = ctx.queue()
    comm = None
    if world > 1:
        box = [U.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        comm = U.Comm(ctx, box[0], rank, world)

    B = args.batch
    stack = U.Stack(ctx, q, shape, enc_id, max_tokens=B, seed=SEED, tp_rank=rank, tp_size=world, comm=comm,
                    flags=U.STACK_FLAG_NCCL_ONLY if args.nccl_only else 0)
    xin = ctx.alloc(B * shape.hidden * 2)
    yout = ctx.alloc(B * stack.local_vocab * 2)
    q.synth_activations(SEED, 77, 0, B * shape.hidden, xin.at(0))
    q.synchronize()

    def barrier():
        q.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing: W warm-up steps, then exactly K steps between two events -------
    for _ in range(args.warmup):
        stack.step(B, xin.at(0), yout.at(0))
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    a = q.signal()
    for _ in range(args.steps):
        stack.step(B, xin.at(0), yout.at(0))
    b = q.signal()
    b.query(3600000)
    ms_total = b.elapsed_ms_since(a)
    a.close()
    b.close()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / args.steps

    # ---- end to end through the host entry point: pinned H2D + step + D2H every step ----------
    x_host = q.download(xin.at(0), (B, shape.hidden), np.uint16)
    y_host = np.empty((B, stack.local_vocab), np.uint16)
    for _ in range(args.warmup):
        stack.step_host_into(x_host, y_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        stack.step_host_into(x_host, y_host)
    q.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()

    wbytes, launches = stack.stats()
    w_algo, a_algo = stack_algorithmic_bytes(shape, enc, B, world)
    assert w_algo == wbytes, (w_algo, wbytes)
    peak, peak_src = peaks()

    line = None
    if rank == 0:
        n_matvec = 4 * shape.layers + 1
        achieved = (w_algo + a_algo) / (ms_step * 1e-3) / 1e9  # GB/s per GPU over the whole step
        line = {
            "metric": "linear-stack decode tokens/s", "value": B / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 accumulate over e4m3 weights and bf16 activations" if enc == "fp8"
            else "f32 accumulate over 4-bit weights (fp16 group scales) and bf16 activations",
            "data": "synthetic",
            "config": {"workload": f"{descr}, batch {B}, tensor-parallel over {world} GPU(s)", "batch": B,
                       "encoding": enc, "layers": shape.layers, "hidden": shape.hidden, "ffn": shape.ffn,
                       "vocab": shape.vocab, "parallelism": f"tp{world}",
                       "l2": "weights streamed per step exceed L2 many times over (no flush needed)",
                       "layers_overridden": bool(args.layers)},
            "e2e": {"value": B * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": B * shape.hidden * 2,
                    "d2h_bytes_per_step": B * stack.local_vocab * 2, "ms_per_step": e2e_s / args.steps * 1e3},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src,
                         "kernel": f"matvec_kernel ({n_matvec} launches per step"
                                   + (f" + {2 * shape.layers} all-reduces" if world > 1 else "") + ")",
                         "algorithmic_bytes_per_step": w_algo + a_algo,
                         "note": "achieved = per-GPU algorithmic bytes of one step / device time of one step"},
        }

    # ---- explanatory figures (rank 0, N = 1 only): single matvec shapes and the CPU port ----------
    stack.close()
    xin.close()
    yout.close()
    if rank == 0 and world == 1 and not args.no_extra:
        extra = {}
        for name, e, n, k, m in (("aq4_m1_k4096_n4096", U.ENCODING_AQ4, 4096, 4096, 1),
                                 ("fp8_m1_k4096_n14336", U.ENCODING_FP8_CHANNEL, 14336, 4096, 1),
                                 ("fp8_m4_k4096_n14336", U.ENCODING_FP8_CHANNEL, 14336, 4096, 4),
                                 ("fp8_m8_k4096_n14336", U.ENCODING_FP8_CHANNEL, 14336, 4096, 8),
                                 ("fp8_m1_k8192_n57344", U.ENCODING_FP8_CHANNEL, 57344, 8192, 1),
                                 ("aq4_m1_k4096_n28672", U.ENCODING_AQ4, 28672, 4096, 1)):
            r = time_matvec_extra(U, ctx, q, e, n, k, m, reps=20, kernel=U.KERNEL_AUTO)
            r["frac_of_peak"] = r["gbs"] / peak
            extra[name] = r
        line["matvec"] = extra
        burst, _, _ = tensor_peaks()
        gemms = {}
        for name, e, mm, n, k in (("aq4_m2048_k4096_n14336", U.ENCODING_AQ4, 2048, 14336, 4096),
                                  ("aq4_m2048_k14336_n4096", U.ENCODING_AQ4, 2048, 4096, 14336),
                                  ("fp8_m2048_k4096_n14336", U.ENCODING_FP8_CHANNEL, 2048, 14336, 4096)):
            r = time_gemm(U, ctx, q, e, mm, n, k, reps=10)
            r["frac_of_peak"] = r["tflops"] / burst
            gemms[name] = r
        line["gemm"] = gemms
        one_pass, elems, threads = cpu_sample(shape, enc, B)
        one_pass()
        passes, spent = [], 0.0
        while spent < 12.0 and len(passes) < 2000:  # about twelve seconds of host work
            passes.append(one_pass())
            spent += passes[-1]
        t = sum(passes) / len(passes)
        scale = shape.weight_elements() / elems
        line["cpu_baseline"] = {
            "value": B / (t * scale), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"one decoder layer of the same widths ({elems} weight elements), {len(passes)} passes in "
                      f"{spent:.1f} s with {threads} threads (mean {t * 1e3:.1f} ms), scaled x{scale:.1f} to the whole "
                      f"stack by weight elements"}
    elif rank == 0:
        line["cpu_baseline"] = None
    if comm is not None:
        comm.close()
    q.close()
    ctx.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

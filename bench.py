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
    return 6650.0, "fallback (6.65 TB/s STREAM-style copy figure; MEASURED_PEAKS.json absent)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (every 50 ms) from before the warm-up on; `stop` keeps
    the samples that fall between `begin()` and `end()`, i.e. inside the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.lines = []  # (host time the line arrived, text)
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.device)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def in_window(self):
        return sum(1 for t, _ in self.lines if self.t0 is not None and self.t0 <= t <= (self.t1 or time.time()) + 0.06)

    def stop(self, window="timed region"):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.06)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for t, line in self.lines:
            if self.t0 is not None and not (self.t0 <= t <= (self.t1 or t) + 0.06):
                continue
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
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


# DRAM traffic of the step's dominant kernel from ncu (dram__bytes_read.sum + dram__bytes_write.sum per launch),
# captured on single-kernel workloads of full shape and scaled to the step by algorithmic bytes: the kernels read
# each weight byte once, so traffic / algorithmic bytes is the same ratio for every matvec of the step.
TRAFFIC_RATIO = {"fp8": 1.007, "aq4": 1.004}  # profiles/matvec_fp8_m1_n57344_k8192.md, matvec_aq4_m1_n28672_k4096.md
TRAFFIC_NOTE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of the matvec kernel on its full-shape single-kernel "
                "workload (profiles/matvec_*.md), scaled to one step by algorithmic bytes")


def stack_traffic(enc, world, algo_bytes):
    return TRAFFIC_RATIO[enc] * algo_bytes


def stack_algorithmic_bytes(shape, enc, batch, tp):
    """Per rank and per step: packed weights + scales + activations read and written by the linears."""
    qd, kvd = shape.q_heads * shape.head_dim, shape.kv_heads * shape.head_dim
    per = (lambda n, k: n * k // 2 + n * k // 64) if enc == "aq4" else (lambda n, k: n * k + 4 * n)
    # (N, K, input bytes per element, output columns, output bytes per element)
    lin = [((qd + 2 * kvd) // tp, shape.hidden, 4, (qd + 2 * kvd) // tp, 2), (shape.hidden, qd // tp, 2, shape.hidden, 4),
           (2 * shape.ffn // tp, shape.hidden, 4, shape.ffn // tp, 2), (shape.hidden, shape.ffn // tp, 2, shape.hidden, 4)]
    w = shape.layers * sum(per(n, k) for n, k, _, _, _ in lin) + per(shape.vocab // tp, shape.hidden)
    a = shape.layers * sum(batch * (k * xi + cols * yo) for n, k, xi, cols, yo in lin)
    a += batch * (shape.hidden * 4 + shape.vocab // tp * 2)
    # glue: one bf16 RMSNorm weight vector per column-parallel linear, one fp32 residual row per row-parallel one,
    # and the bf16 -> fp32 copy that starts the residual stream
    a += (2 * shape.layers + 1) * shape.hidden * 2 + 2 * shape.layers * batch * shape.hidden * 4 + batch * shape.hidden * 6
    return w, a


class CpuStack:
    """The plain-C port (oracle/oracle_c.c, fp32 accumulate, OpenMP over output channels) running one decode step
    of the linear stack on the host: per layer rmsnorm -> QKV -> O + residual -> rmsnorm -> gate|up -> swiglu ->
    down + residual, then rmsnorm -> LM head.  All layers stream the SAME layer's weight bytes (one layer of
    random codes is held in host memory, 0.86 GB at 70B widths: far beyond any CPU cache, so every pass still
    streams from DRAM); the LM head has its own.  The reference project has no CPU (or any) implementation of this
    path: this is `kind: "port"`."""

    def __init__(self, shape, enc, batch, threads=None):
        import oracle_c as oc
        self.oc, self.shape, self.enc, self.batch = oc, shape, enc, batch
        if threads is None:
            threads = os.cpu_count() or 1  # torch.distributed.run exports OMP_NUM_THREADS=1: ask for the cores explicitly
        oc.set_num_threads(threads)
        self.threads = oc.num_threads()
        rng = np.random.default_rng(SEED)
        qd, kvd = shape.q_heads * shape.head_dim, shape.kv_heads * shape.head_dim
        self.qd = qd
        dims = [(qd + 2 * kvd, shape.hidden), (shape.hidden, qd), (2 * shape.ffn, shape.hidden), (shape.hidden, shape.ffn)]

        def weight(n, k):  # random codes (timing only): any byte is a valid AQ4 pair; 0xF7 keeps e4m3 off its NaN codes
            if enc == "aq4":
                raw = np.frombuffer(rng.bytes(n * (k // 2)), np.uint8).reshape(n, k // 2)
                return raw, np.full((n, k // 128), 0.003, np.float16)
            raw = np.frombuffer(rng.bytes(n * k), np.uint8).reshape(n, k) & np.uint8(0xF7)
            return raw, np.full(n, 1e-4, np.float32)

        self.layer = [weight(n, k) for n, k in dims]
        self.head = weight(shape.vocab, shape.hidden)
        self.layer_elems = sum(n * k for n, k in dims)
        self.gamma = np.ones(shape.hidden, np.float32)
        self.x = (oc.synth_activations_bits(SEED, 5000, batch, shape.hidden).astype(np.uint32) << 16).view(np.float32)

    def _lin(self, x_f32, w, want):
        import oracle as o
        bits = o.f32_to_bf16_bits(x_f32).reshape(x_f32.shape)
        return (self.oc.linear_aq4 if self.enc == "aq4" else self.oc.linear_fp8)(bits, w[0], w[1], want=want)

    @staticmethod
    def _rms(h, gamma):
        r = 1.0 / np.sqrt((h.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
        return (h * r * gamma).astype(np.float32)

    def layer_pass(self, h):
        qkv = self._lin(self._rms(h, self.gamma), self.layer[0], "bf16")
        h = h + self._lin(qkv[:, :self.qd], self.layer[1], "f32")
        gu = self._lin(self._rms(h, self.gamma), self.layer[2], "bf16")
        f = gu.shape[1] // 2
        act = gu[:, :f] / (1.0 + np.exp(-gu[:, :f])) * gu[:, f:]
        return h + self._lin(act.astype(np.float32), self.layer[3], "f32")

    def step(self, layers=None):
        """One whole decode step (all layers + LM head); returns seconds."""
        t0 = time.perf_counter()
        h = self.x.copy()
        for _ in range(self.shape.layers if layers is None else layers):
            h = self.layer_pass(h)
            h *= np.float32(1.0 / max(1.0, float(np.abs(h).max())))  # keeps the synthetic residual stream bounded
        self._lin(self._rms(h, self.gamma), self.head, "bf16")
        return time.perf_counter() - t0


def cpu_single_ops(threads_all):
    """The plain-C port on the single-op benchmark configurations (1: AQ4 matvec 4096x4096; 2: FP8 matvec
    14336x4096, M = 1/4/8; 3: AQ4 GEMM 14336x4096 and 4096x14336 on a 64-token sample of the 2048 tokens, scaled
    linearly in M), once with every host core and once on a single thread.  Seconds per call."""
    import oracle_c as oc
    rng = np.random.default_rng(SEED + 1)
    out = {}

    def weight(enc, n, k):
        if enc == "aq4":
            return np.frombuffer(rng.bytes(n * (k // 2)), np.uint8).reshape(n, k // 2), np.full((n, k // 128), 0.003, np.float16)
        return np.frombuffer(rng.bytes(n * k), np.uint8).reshape(n, k) & np.uint8(0xF7), np.full(n, 1e-4, np.float32)

    cases = [("config1_aq4_m1_k4096_n4096", "aq4", 1, 4096, 4096, 1.0), ("config2_fp8_m1_k4096_n14336", "fp8", 1, 14336, 4096, 1.0),
             ("config2_fp8_m4_k4096_n14336", "fp8", 4, 14336, 4096, 1.0), ("config2_fp8_m8_k4096_n14336", "fp8", 8, 14336, 4096, 1.0),
             ("config3_aq4_m2048_k4096_n14336", "aq4", 64, 14336, 4096, 32.0), ("config3_aq4_m2048_k14336_n4096", "aq4", 64, 4096, 14336, 32.0)]
    for name, enc, m, n, k, scale in cases:
        w = weight(enc, n, k)
        x = oc.synth_activations_bits(SEED, 6000 + m, m, k)
        fn = oc.linear_aq4 if enc == "aq4" else oc.linear_fp8
        rec = {}
        for label, threads in (("all_cores", threads_all), ("single_thread", 1)):
            oc.set_num_threads(threads)
            fn(x, w[0], w[1])
            reps = 3 if label == "all_cores" else 1
            t0 = time.perf_counter()
            for _ in range(reps):
                fn(x, w[0], w[1])
            rec[label + "_ms"] = (time.perf_counter() - t0) / reps * 1e3 * scale
        rec["cores"] = threads_all
        if scale != 1.0:
            rec["sample"] = f"{m} of the tokens, scaled x{scale:.0f}"
        out[name] = rec
    oc.set_num_threads(threads_all)
    return out


def reference_config(args, shape, enc, descr, world):
    """The `config` object both arms print (the driver compares them key by key)."""
    return {"workload": f"{descr}, batch {args.batch}, tensor-parallel over {world} GPU(s)", "batch": args.batch,
            "encoding": enc, "layers": shape.layers, "hidden": shape.hidden, "ffn": shape.ffn,
            "vocab": shape.vocab, "parallelism": f"tp{world}",
            "l2": "weights streamed per step exceed L2 many times over (no flush needed)",
            "layers_overridden": bool(args.layers)}


def run_reference(args, shape, enc, descr):
    """The reference project has no CPU (or any) implementation of this path, so the reference arm times this
    repository's plain-C port of the format spec on the host cores: every step executes ALL layers and the LM head
    (nothing is extrapolated), with every host core, whatever OMP_NUM_THREADS the launcher exported."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuStack(shape, enc, args.batch)
    for _ in range(args.warmup):
        cpu.step()
    times = [cpu.step() for _ in range(args.steps)]
    t = sum(times) / len(times)
    value = args.batch / t
    sample = (f"whole steps: {shape.layers} layer passes (QKV, O, gate+up, down with their glue) + LM head per step, "
              f"{args.steps} timed steps of {t:.2f} s on {cpu.threads} threads; the layers share one layer's weight bytes "
              f"({cpu.layer_elems} elements, streamed from DRAM every pass)")
    line = {
        "impl": "reference", "metric": "linear-stack decode tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 accumulate over e4m3 weights and bf16 activations" if enc == "fp8"
        else "f32 accumulate over 4-bit weights (fp16 group scales) and bf16 activations",
        "data": "synthetic",
        "config": reference_config(args, shape, enc, descr, args.gpus),
        "note": "CPU port of the spec on the host cores (the reference has no implementation of this path); "
                "the GPU count only names the arm's configuration",
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cpu.threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def tp_check(U, ctx, q, comm, dist, shape, enc, enc_id, rank, world):
    """Before anything is timed at N > 1: a 2-layer stack of the benchmark's widths (vocabulary cut to 16032 to
    bound the host work) at the same tensor-parallel degree runs one step with the fused all-reduce and one with
    ncclAllReduce; rank 0 walks the oracle chain once (plain-C port, all host threads) and checks
      * every row-parallel sum (O and down of both layers) at the stated tolerance, against the full-K oracle linear
        applied to the DEVICE's own inputs gathered from the ranks, plus the residual, and
      * every rank's slice of the logits against the chain's, as rms error relative to the rms of the logits
        (a chain of bf16 roundings is only reproducible to the 1-ulp level end to end: bound 2 %).
    The oracle is the checker here, outside every timed region."""
    import oracle as o
    import oracle_c as oc
    chk = U.StackShape(2, shape.hidden, shape.q_heads, shape.kv_heads, shape.head_dim, shape.ffn, 16032)
    qd, kvd = chk.q_heads * chk.head_dim, chk.kv_heads * chk.head_dim
    x = o.synth_activations(SEED, 78, 1, chk.hidden)
    xb = o.f32_to_bf16_bits(x).reshape(1, chk.hidden)
    got = {}
    for mode, flags in (("push", 0), ("nccl", U.STACK_FLAG_NCCL_ONLY)):
        st = U.Stack(ctx, q, chk, enc_id, max_tokens=1, seed=SEED, tp_rank=rank, tp_size=world, comm=comm,
                     flags=flags | U.STACK_FLAG_KEEP_ACTIVATIONS)
        for _ in range(2):  # the second step replays the captured graph
            logits = st.step_host(xb)
        rec = {"logits": logits}
        for layer in range(chk.layers):
            for which, kl, cols in ((U.LINEAR_O, qd // world, (qd + 2 * kvd) // world), (U.LINEAR_DOWN, chk.ffn // world, chk.ffn // world)):
                info = st.linear_info(layer, which)
                rec[(layer, which)] = (q.download(info.last_input, (1, cols), np.uint16)[:, :kl].copy(),
                                       q.download(info.last_residual, (1, chk.hidden), np.float32),
                                       q.download(info.last_output, (1, chk.hidden), np.float32))
        _, rec["launches"] = st.stats()
        st.close()
        gathered = [None] * world
        dist.all_gather_object(gathered, rec)
        got[mode] = gathered
    result = None
    if rank == 0:
        oc.set_num_threads(os.cpu_count() or 1)

        def weight(layer, which, n, k):
            w = oc.synth_weights(SEED, o.stack_tensor_id(layer, which), n, k)
            return oc.aq4_quantize(w) if enc == "aq4" else oc.fp8_quantize(w)

        def lin(x_f32, w, want):
            bits = o.f32_to_bf16_bits(np.ascontiguousarray(x_f32, np.float32)).reshape(x_f32.shape)
            return (oc.linear_aq4 if enc == "aq4" else oc.linear_fp8)(bits, w[0], w[1], want=want)

        worst = {m: {"max_rel_floored": 0.0, "mean_abs": 0.0} for m in got}
        h = x.astype(np.float32)
        for layer in range(chk.layers):
            g1, g2 = o.stack_gamma(SEED, layer, o.STACK_QKV, chk.hidden), o.stack_gamma(SEED, layer, o.STACK_GATE_UP, chk.hidden)
            qkv = lin(o.rmsnorm(o.bf16_round(h), 1e-5, g1), weight(layer, o.STACK_QKV, qd + 2 * kvd, chk.hidden), "bf16")
            wo = weight(layer, o.STACK_O, chk.hidden, qd)
            h1 = (h + lin(qkv[:, :qd], wo, "f32")).astype(np.float32)
            gu = o.swiglu(lin(o.rmsnorm(o.bf16_round(h1), 1e-5, g2), weight(layer, o.STACK_GATE_UP, 2 * chk.ffn, chk.hidden), "bf16"))
            wd = weight(layer, o.STACK_DOWN, chk.hidden, chk.ffn)
            h = (h1 + lin(gu, wd, "f32")).astype(np.float32)
            for mode, ranks in got.items():
                for which, w in ((U.LINEAR_O, wo), (U.LINEAR_DOWN, wd)):
                    xin = o.bf16_bits_to_f32(np.concatenate([r[(layer, which)][0] for r in ranks], axis=1))
                    resid, out = ranks[0][(layer, which)][1], ranks[0][(layer, which)][2]
                    stt = o.error_stats(out, (resid + lin(xin, w, "f32")).astype(np.float32))
                    for key in worst[mode]:
                        worst[mode][key] = max(worst[mode][key], stt[key] if stt["nan"] == 0 and stt["inf"] == 0 else float("inf"))
        ref = lin(o.rmsnorm(o.bf16_round(h), 1e-5, o.stack_gamma(SEED, 0, o.STACK_LM_HEAD, chk.hidden)),
                  weight(0, o.STACK_LM_HEAD, chk.vocab, chk.hidden), "bf16")
        result = {"stack": "2 layers of the benchmark's widths, vocabulary 16032, 1 token", "modes": {}}
        ok = True
        for mode, ranks in got.items():
            dev = np.concatenate([o.bf16_bits_to_f32(r["logits"]) for r in ranks], axis=1)
            rel = float(np.sqrt(np.mean((dev - ref) ** 2)) / np.sqrt(np.mean(ref ** 2)))
            fine = bool(np.isfinite(dev).all() and rel < 0.02 and worst[mode]["max_rel_floored"] <= 1e-2
                        and worst[mode]["mean_abs"] <= 1e-3)
            result["modes"][mode] = {"max_rel_floored": worst[mode]["max_rel_floored"], "mean_abs": worst[mode]["mean_abs"],
                                     "logits_rel_rms": rel, "launches_per_step": ranks[0]["launches"], "pass": fine}
            ok = ok and fine
        result.update({"mode": "push+nccl", "max_rel_floored": max(v["max_rel_floored"] for v in result["modes"].values()),
                       "mean_abs": max(v["mean_abs"] for v in result["modes"].values()), "pass": ok})
    box = [result]
    dist.broadcast_object_list(box, src=0)
    return box[0]


def time_stack(stack, q, B, xin, yout, steps, warmup):
    """Device time per step (ms) of `steps` steps after `warmup`, between two events on the stack's queue."""
    for _ in range(warmup):
        stack.step(B, xin.at(0), yout.at(0))
    q.synchronize()
    a = q.signal()
    for _ in range(steps):
        stack.step(B, xin.at(0), yout.at(0))
    b = q.signal()
    b.query(3600000)
    ms = b.elapsed_ms_since(a) / steps
    a.close()
    b.close()
    return ms


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
    return 1590.0, 1400.0, "fallback (1.59 PFLOP/s cuBLAS bf16 burst figure; MEASURED_PEAKS.json absent)"


def time_gemm(U, ctx, q, enc_id, m, n, k, reps):
    """Device time of one fused-dequant GEMM launch (tcgen05 path), activations [m,k] bf16 resident in HBM.
    Launches alternate between two copies of the weights and two outputs, so the operands and results of
    consecutive launches (together well over the 126 MB L2) are never the same."""
    vb, sb = U.weight_bytes(enc_id, n, k)
    src = ctx.alloc(n * k * 4)
    q.synth_weights(SEED, 4300, 0, n * k, 0.02, src.at(0))
    sets = []
    for _ in range(2):
        v, s = ctx.alloc(vb), ctx.alloc(sb)
        wd = U.weight_desc(enc_id, n, k, v.at(0), s.at(0))
        q.quantize(src.at(0), wd)
        sets.append((v, s, wd, ctx.alloc(m * n * 2)))
    src.close()
    xb = ctx.alloc(m * k * 2)
    q.synth_activations(SEED, 4301, 0, m * k, xb.at(0))
    descs = [U.linear_desc(wd, m, xb.at(0), yb.at(0), kernel=U.KERNEL_GEMM) for (_, _, wd, yb) in sets]
    for i in range(4):
        q.linear_enqueue(descs[i & 1])
    q.synchronize()
    a = q.signal()
    for i in range(reps):
        q.linear_enqueue(descs[i & 1])
    b = q.signal()
    b.query(600000)
    ms = b.elapsed_ms_since(a) / reps
    a.close()
    b.close()
    for (v, s, _, yb) in sets:
        for buf in (v, s, yb):
            buf.close()
    xb.close()
    flops = 2.0 * m * n * k
    return {"us_per_launch": ms * 1e3, "tflops": flops / (ms * 1e-3) / 1e12, "flops": flops,
            "weight_gbs": (vb + sb) / (ms * 1e-3) / 1e9,
            "l2": "two weight copies and two outputs alternate between launches"}


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
        "steps": args.steps, "warmup": 4, "ms_per_step": r["us_per_launch"] / 1e3, "higher_is_better": True,
        "config": {"workload": f"{args.enc} GEMM M={args.batch} N={args.n} K={args.k}"},
        "roofline": {"bound": "tensor", "achieved": r["tflops"], "peak": burst, "unit": "TFLOP/s",
                     "frac": r["tflops"] / burst, "traffic": None, "peak_source": src,
                     "frac_of_sustained": r["tflops"] / sustained, "frac_of_nominal_2250": r["tflops"] / 2250.0,
                     "weight_stream_gbs": r["weight_gbs"]},
        "gpu_launches": 2 * (max(args.steps, 1) + 4)}), flush=True)
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


def run_single_gather(U, args):
    """The consumer half of the fused all-reduce alone, on one GPU: the slots of `--ranks` ranks are filled once
    (values and tags in place), then a QKV-shaped linear (N = --n, K = --k, RMSNorm with weight, residual) gathers
    them `--steps` times per graph replay over enough weight copies to exceed 2x L2.  Shows what the gather costs
    on top of the plain matvec of the same shape (no NVLink and no skew between ranks in this figure)."""
    ctx = U.Context(0)
    q = ctx.queue()
    enc_id = U.ENCODING_AQ4 if args.enc == "aq4" else U.ENCODING_FP8_CHANNEL
    n, k, m, ranks = args.n, args.k, args.batch, args.ranks
    vb, sb = U.weight_bytes(enc_id, n, k)
    copies = max(2, int(2 * 130e6 // (vb + sb)) + 1)
    src = ctx.alloc(n * k * 4)
    q.synth_weights(SEED, 4242, 0, n * k, 0.02, src.at(0))
    stride = m * k * 8
    slots = ctx.alloc(ranks * stride)
    pairs = np.zeros((ranks, m * k, 2), np.uint32)
    pairs[:, :, 0] = (np.random.default_rng(SEED).standard_normal((ranks, m * k)).astype(np.float32) / np.float32(ranks)).view(np.uint32)
    pairs[:, :, 1] = 9
    q.upload(slots.at(0), pairs)
    resid, gam = ctx.alloc(m * k * 4), ctx.alloc(k * 2)
    q.synth_weights(SEED, 4250, 0, m * k, 1.0, resid.at(0))
    q.fill(gam.at(0), 0x3F, k * 2)  # bf16 0x3F3F = 0.746
    xdummy, yb = ctx.alloc(m * k * 4), ctx.alloc(m * n * 2)
    bufs, descs = [], []
    for _ in range(copies):
        v, sc = ctx.alloc(vb), ctx.alloc(sb)
        wd = U.weight_desc(enc_id, n, k, v.at(0), sc.at(0))
        q.quantize(src.at(0), wd)
        bufs += [v, sc]
        descs.append(U.linear_desc(wd, m, xdummy.at(0), yb.at(0), input_dtype=U.DTYPE_F32, prologue=U.PROLOGUE_RMSNORM,
                                   norm_weight=gam.at(0), residual=resid.at(0)))
    sl = U.slots_desc(slots.at(0), stride, ranks, tag=9, gather=1 if args.gather == "cluster" else 0)
    q.linear_enqueue_reduced(descs[0], sl)
    assert q.synchronize().device_flags == 0
    q.capture_begin()
    for d in descs:
        q.linear_enqueue_reduced(d, sl)
    g = q.capture_end()
    for _ in range(3):
        g.launch(q)
    q.synchronize()
    a = q.signal()
    for _ in range(max(args.steps, 1)):
        g.launch(q)
    b = q.signal()
    b.query(600000)
    us = b.elapsed_ms_since(a) * 1e3 / (max(args.steps, 1) * copies)
    a.close()
    b.close()
    g.close()
    algo = vb + sb + ranks * m * k * 8 + m * k * 4 + m * n * 2
    peak, peak_src = peaks()
    print(json.dumps({
        "metric": "gathering matvec HBM GB/s", "value": algo / us / 1e3, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": 3, "ms_per_step": us * copies / 1e3, "higher_is_better": True,
        "config": {"workload": f"{args.enc} matvec M={m} N={n} K={k} gathering {ranks} ranks' slots per {args.gather}",
                   "weight_copies": copies},
        "roofline": {"bound": "hbm", "achieved": algo / us / 1e3, "peak": peak, "unit": "GB/s", "frac": algo / us / 1e3 / peak,
                     "traffic": None, "peak_source": peak_src, "us_per_launch": us, "algorithmic_bytes": algo},
        "gpu_launches": copies * (max(args.steps, 1) + 4)}), flush=True)
    for buf in bufs + [src, slots, resid, gam, xdummy, yb]:
        buf.close()
    q.close()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--workload", default="stack70b-fp8", choices=sorted(WORKLOADS) + ["matvec", "gemm", "gather"])
    ap.add_argument("--ranks", type=int, default=8, help="gather workload: ranks whose slots are summed")
    ap.add_argument("--enc", default="fp8", choices=["fp8", "aq4"], help="matvec workload: weight encoding")
    ap.add_argument("--kernel", default="auto", choices=["auto", "matvec", "gemm"],
                    help="matvec workload: kernel behind the linear op (auto: by token count)")
    ap.add_argument("--n", type=int, default=57344, help="matvec workload: output channels")
    ap.add_argument("--k", type=int, default=8192, help="matvec workload: reduction length")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; the line says so)")
    ap.add_argument("--no-extra", action="store_true", help="skip the single-matvec figures and the CPU baseline")
    ap.add_argument("--nccl-only", action="store_true", help="sum over ranks with ncclAllReduce instead of the fused peer-memory push")
    ap.add_argument("--gather", default="auto", choices=["auto", "block", "cluster"],
                    help="fused all-reduce: how the consuming kernels gather the ranks' slots")
    ap.add_argument("--no-check", action="store_true", help="skip the tensor-parallel parity check that precedes the timed region")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    import ullm_cuda as U

    if args.workload == "matvec":
        run_single_matvec(U, args)
        return
    if args.workload == "gemm":
        run_single_gemm(U, args)
        return
    if args.workload == "gather":
        run_single_gather(U, args)
        return
    shape_name, enc, descr = WORKLOADS[args.workload]
    shape = getattr(U, shape_name)
    if args.layers:
        shape = U.StackShape(args.layers, shape.hidden, shape.q_heads, shape.kv_heads, shape.head_dim, shape.ffn, shape.vocab)
    if args.impl == "reference":
        run_reference(args, shape, enc, descr)
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
    check = None
    if world > 1 and not args.no_check:
        check = tp_check(U, ctx, q, comm, dist, shape, enc, enc_id, rank, world)
        if not check["pass"]:
            if rank == 0:
                print(json.dumps({"check": check, "error": "tensor-parallel results differ from the oracle"}), flush=True)
            raise SystemExit(3)
    extras_on = rank == 0 and world == 1 and not args.no_extra
    flags = (U.STACK_FLAG_NCCL_ONLY if args.nccl_only else 0) | {"auto": 0, "block": U.STACK_FLAG_GATHER_PER_BLOCK,
                                                                  "cluster": U.STACK_FLAG_GATHER_PER_CLUSTER}[args.gather]
    # at N = 1 the same stack also serves the batch-32 figure of the extra block
    stack = U.Stack(ctx, q, shape, enc_id, max_tokens=max(B, 32) if extras_on and args.workload == "stack70b-fp8" else B,
                    seed=SEED, tp_rank=rank, tp_size=world, comm=comm, flags=flags)
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
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # before the warm-up, so that nvidia-smi is already looping when the timed region begins
    for _ in range(args.warmup):
        stack.step(B, xin.at(0), yout.at(0))
    barrier()
    q.synchronize()
    sampler.begin()
    a = q.signal()
    for _ in range(args.steps):
        stack.step(B, xin.at(0), yout.at(0))
    b = q.signal()
    b.query(3600000)
    sampler.end()
    ms_total = b.elapsed_ms_since(a)
    a.close()
    b.close()
    barrier()
    clock_window = "timed region"
    ms_total = max_over_ranks(ms_total)
    short = max_over_ranks(1.0 if (rank == 0 and sampler.proc is not None and sampler.in_window() < 2) else 0.0)
    if short > 0.0:
        # the timed region was shorter than two sampling periods: every rank keeps the same step running (untimed) for
        # about 0.6 s and rank 0 reads the clocks under that load instead
        clock_window = "the same step repeated right after the timed region (which was shorter than two samples)"
        n_extra = int(min(400, max(8, 600.0 / (ms_total / args.steps))))
        sampler.begin()
        for _ in range(n_extra):
            stack.step(B, xin.at(0), yout.at(0))
        q.synchronize()
        sampler.end()
        barrier()
    clocks = sampler.stop(clock_window) if rank == 0 else None
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
            "config": reference_config(args, shape, enc, descr, world),
            "check": check,
            "e2e": {"value": B * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": B * shape.hidden * 2,
                    "d2h_bytes_per_step": B * stack.local_vocab * 2, "ms_per_step": e2e_s / args.steps * 1e3},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": stack_traffic(enc, world, w_algo + a_algo), "peak_source": peak_src,
                         "traffic_source": TRAFFIC_NOTE,
                         "kernel": f"matvec_kernel ({n_matvec} launches per step"
                                   + (f" + {2 * shape.layers} all-reduces" if world > 1 else "") + ")",
                         "algorithmic_bytes_per_step": w_algo + a_algo,
                         "note": "achieved = per-GPU algorithmic bytes of one step / device time of one step"},
        }

    # ---- explanatory figures (rank 0, N = 1 only): the other benchmark configurations, single shapes, the CPU port
    stacks = {}
    if extras_on and args.workload == "stack70b-fp8":
        x32, y32 = ctx.alloc(32 * shape.hidden * 2), ctx.alloc(32 * stack.local_vocab * 2)
        q.synth_activations(SEED, 79, 0, 32 * shape.hidden, x32.at(0))
        ms = time_stack(stack, q, 32, x32, y32, 10, 3)
        stacks["stack70b_fp8_batch32"] = {"ms_per_step": ms, "tokens_per_s": 32 / (ms * 1e-3)}
        x32.close()
        y32.close()
    stack.close()
    xin.close()
    yout.close()
    if extras_on:
        if args.workload == "stack70b-fp8":
            # benchmark config 5, prefill: the same stack with 4096 tokens in one step (tensor-core kernels throughout)
            try:
                T = 4096
                sp = U.Stack(ctx, q, shape, enc_id, max_tokens=T, seed=SEED)
                xp, yp = ctx.alloc(T * shape.hidden * 2), ctx.alloc(T * sp.local_vocab * 2)
                q.synth_activations(SEED, 81, 0, T * shape.hidden, xp.at(0))
                ms = time_stack(sp, q, T, xp, yp, 2, 1)
                flops = 2.0 * T * shape.weight_elements()
                burst_p, _, _ = tensor_peaks()
                stacks["stack70b_fp8_prefill4096"] = {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
                                                      "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / burst_p}
                sp.close()
                xp.close()
                yp.close()
            except Exception as exc:  # an explanatory figure must not take the headline line down with it
                stacks["stack70b_fp8_prefill4096"] = {"error": str(exc)[:200]}
            s8 = U.Stack(ctx, q, U.LLAMA3_8B, U.ENCODING_AQ4, max_tokens=64, seed=SEED)
            x8, y8 = ctx.alloc(64 * 4096 * 2), ctx.alloc(64 * s8.local_vocab * 2)
            q.synth_activations(SEED, 80, 0, 64 * 4096, x8.at(0))
            w8, _ = s8.stats()
            for b8 in (1, 16, 64):
                ms = time_stack(s8, q, b8, x8, y8, 20, 3)
                stacks[f"stack8b_aq4_batch{b8}"] = {"ms_per_step": ms, "tokens_per_s": b8 / (ms * 1e-3),
                                                    "weight_gbs": w8 / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": w8 / (ms * 1e-3) / 1e9 / peak}
            s8.close()
            x8.close()
            y8.close()
        line["stacks"] = stacks
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
                                  ("fp8_m2048_k4096_n14336", U.ENCODING_FP8_CHANNEL, 2048, 14336, 4096),
                                  ("fp8_m2048_k14336_n4096", U.ENCODING_FP8_CHANNEL, 2048, 4096, 14336),
                                  ("fp8_m4096_k8192_n57344", U.ENCODING_FP8_CHANNEL, 4096, 57344, 8192)):
            r = time_gemm(U, ctx, q, e, mm, n, k, reps=10)
            r["frac_of_peak"] = r["tflops"] / burst
            gemms[name] = r
        line["gemm"] = gemms
        # the CPU port beside it: a bounded sample (about twelve seconds) of the same step with every host core, and
        # one decoder layer on a single core
        cpu = CpuStack(shape, enc, B)
        h = cpu.x.copy()
        cpu.layer_pass(h)
        passes, spent = [], 0.0
        while spent < 12.0 and len(passes) < 4000:
            t0 = time.perf_counter()
            cpu.layer_pass(h)
            passes.append(time.perf_counter() - t0)
            spent += passes[-1]
        t = sum(passes) / len(passes)
        scale = shape.weight_elements() / cpu.layer_elems
        cpu.oc.set_num_threads(1)
        t0 = time.perf_counter()
        cpu.layer_pass(h)
        t1 = time.perf_counter() - t0
        line["cpu_single_ops"] = cpu_single_ops(cpu.threads)
        line["cpu_baseline"] = {
            "value": B / (t * scale), "unit": "tokens/s", "cores": cpu.threads, "kind": "port",
            "single_thread_value": B / (t1 * scale),
            "sample": f"one decoder layer of the same widths with its glue ({cpu.layer_elems} weight elements), {len(passes)} "
                      f"passes in {spent:.1f} s with {cpu.threads} threads (mean {t * 1e3:.1f} ms; one pass on a single thread "
                      f"{t1 * 1e3:.0f} ms), scaled x{scale:.1f} to the whole stack by weight elements; the reference arm "
                      f"(--impl reference) executes whole steps instead"}
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

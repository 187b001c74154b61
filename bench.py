#!/usr/bin/env python
"""Benchmark of the docc library-node hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload softmax|gemm_f64|conv_f32|conv_bf16|attention|attention_causal|block_f32|block_bf16]
                    [--no-extras]

Prints ONE JSON line. The headline workload (default) is BASELINE config 2: row softmax over a
fp32 [8192, 4096] tensor, reported as algorithmic HBM GB/s (one read + one write of the tensor).
A "step" is one pass of the node over one batch of synthetic input. With --gpus N every rank
processes its own batch (weak scaling over independent units, no data-path collective); for the sharded
configurations (conv, attention, encoder block) the line's extras also carry the split-and-gather reading:
ONE configuration split across the ranks, each step ending with the in-place NCCL all-gather of the output
shards (``--strong`` makes that the headline of a single ``--workload``).

``--impl reference`` times the CPU restatement of the reference's own expansion of the node
(oracle/, OpenMP over the outermost map as docc's openmp target schedules it) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from docc_b200.sharding import GatherPlan  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum per launch of each workload's dominant kernel, from the ncu captures
# (isolated launches: part of the write-back is still in L2 when the kernel ends, which is why the softmax figure is
# below its 268 MB of algorithmic bytes)
NCU_TRAFFIC_BYTES = {"softmax": 213.9e6, "gemm_bf16": 1001.2e6, "conv_bf16": 14.9e6, "conv_f32": 28.6e6, "attention": 243.7e6, "attention_causal": 566.4e6,
                     "gemm_f64": 16.0e6}

# Sharded workloads (conv, attention, encoder block) at N > 1 GPUs are read two ways. Weak (the headline `value`): every
# GPU runs the whole configuration on its own data and nothing is exchanged. Split-and-gather (`--strong`, and the
# `split_gather` list of the line at N > 1): ONE configuration is split over the GPUs and every step ends with the NCCL
# all-gather of the output shards, in place and chunked so that it overlaps the kernels of the next chunk.
STRONG = False
# Chunks per step of the split-and-gather mode. More than one overlaps the gather of a chunk with the kernels of the next,
# but at these sizes it costs more than it hides: half-size calls fill the 148 SMs worse (attention: 256 work items per
# call are 1.7 waves) and every extra launch is paid on the host. Measured at 2 GPUs, encoder block bf16: 0.43 ms with
# two chunks against 0.29 ms with one.
GATHER_CHUNKS = 1

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# cuBLAS DGEMM 8192^3 through torch on this pool's B200, measured by the builder: tcgen05 has no fp64 kind, so this is
# the practical ceiling config 1 is held against (not in MEASURED_PEAKS.json)
FP64_TFLOPS_BUILDER_MEASURED = 35.5

WORKLOAD_TEXT = {
    "softmax": "softmax fp32 [8192,4096] axis=-1 (BASELINE config 2)",
    "gemm_f64": "GEMM fp64 1000x1000x1000 (BASELINE config 1)",
}


def headline_config():
    """The `config` object of the headline line; both arms print exactly this."""
    return {"workload": WORKLOAD_TEXT["softmax"], "rows_per_gpu": 8192, "cols": 4096,
            "l2": "inputs larger than L2 and rotated over 4 buffer pairs"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bind_near_gpu(device_index):
    """Restricts this process to the CPU cores of the NUMA node its GPU hangs off (read from sysfs), so that pinned host
    buffers are first touched, and the copy threads run, next to the GPU's PCIe root. With eight ranks on a two-socket
    host the end-to-end path (H2D + kernel + D2H through pinned memory) is bounded by host memory traffic; unbound ranks
    all land on one socket. Best effort: returns a description, never raises."""
    info = {"bound": False}
    try:
        out = subprocess.run(["nvidia-smi", f"--id={device_index}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=10).stdout.strip()
        bus = out.lower()
        if bus.startswith("00000000:"):
            bus = bus[4:]  # sysfs uses a 4-digit domain
        node_path = f"/sys/bus/pci/devices/{bus}/numa_node"
        node = int(open(node_path).read().strip())
        info["pci"], info["numa_node"] = bus, node
        if node < 0:
            return info
        cpus = []
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.extend(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["bound"], info["cpus"] = True, len(allowed)
    except Exception as exc:
        info["error"] = f"{type(exc).__name__}: {exc}"[:120]
    return info


# ------------------------------------------------------------------------------------------------------
# workloads: each returns a dict with a `step()` closure over device-resident inputs, the algorithmic
# work per step and the roofline that bounds it
# ------------------------------------------------------------------------------------------------------
def make_workload(name, torch, ops, rank, world, strong=False):
    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = measured_peaks()
    g = torch.Generator(device="cpu")

    if name == "softmax":
        rows, cols = 8192, 4096
        g.manual_seed(1 + rank)
        n_buf = 4  # 4 x (134 MB in + 134 MB out): consecutive steps never find their input in the 126 MB L2
        xs = [(3 * torch.randn(rows, cols, generator=g)).to(dev) for _ in range(n_buf)]
        ys = [torch.empty_like(x) for x in xs]
        shape = ops._arr((rows, cols))
        axes = ops._arr((1,))
        state = {"i": 0}

        def step():
            i = state["i"] % n_buf
            state["i"] += 1
            ops.call("docc_b200_softmax", ord("s"), 2, shape, 1, axes, ops._ptr(xs[i]), ops._ptr(ys[i]), 0)

        units = 2 * rows * cols * 4  # bytes: one read + one write
        return dict(step=step, units=units, unit="GB/s", scale=1e-9, metric="softmax_hbm_gbs", dtype="f32",
                    bound="hbm", peak=peaks["hbm_gbs"], launches_per_step=1,
                    config=headline_config(),
                    host_inputs=lambda: [(3 * torch.randn(rows, cols, generator=g))], kind="softmax",
                    h2d=rows * cols * 4, d2h=rows * cols * 4)

    if name == "gemm_f64":
        # 93 us steps: timed back to back over eight operand / result sets (24 MB each, 192 MB in all: larger than L2), for the
        # reason given at the conv workloads
        rs = np.random.RandomState(0)
        n_sets = 8
        sets = []
        for _ in range(n_sets):
            a = torch.from_numpy(rs.rand(1000, 1000)).to(dev)
            b = torch.from_numpy(rs.rand(1000, 1000)).to(dev)
            sets.append((a, b, torch.empty(1000, 1000, dtype=torch.float64, device=dev)))
        state = {"i": 0}

        def step():
            a, b, c = sets[state["i"] % n_sets]
            state["i"] += 1
            ops.gemm(a, b, c)

        return dict(step=step, units=2 * 1000 ** 3, unit="TFLOP/s", scale=1e-12, metric="gemm_fp64_tflops", dtype="f64",
                    bound="tensor", peak=FP64_TFLOPS_BUILDER_MEASURED, peak_source="of the builder-measured cuBLAS DGEMM 8192^3 rate",
                    launches_per_step=1, steps_scale=20,
                    config={"workload": WORKLOAD_TEXT["gemm_f64"], "l2": "operands and results rotated over 8 sets, larger than L2"},
                    kind="gemm", replicas_only=True)

    if name in ("gemm_bf16", "gemm_f32"):
        # not a BASELINE config: the engine's own large-GEMM point, next to cuBLAS-class numbers
        n = 8192
        dt = torch.bfloat16 if name == "gemm_bf16" else torch.float32
        g.manual_seed(6)
        a = torch.randn(n, n, generator=g).to(dt).to(dev)
        b = torch.randn(n, n, generator=g).to(dt).to(dev)  # [N, K]: torch Linear layout
        c = torch.empty(n, n, dtype=dt, device=dev)

        def step():
            ops.gemm(a, b, c, transb=True)

        return dict(step=step, units=2 * n ** 3, unit="TFLOP/s", scale=1e-12, metric=name + "_tflops",
                    dtype="bf16" if name == "gemm_bf16" else "f32(split-bf16x3)", bound="tensor",
                    peak=peaks["bf16_tflops"] / (1 if name == "gemm_bf16" else 3), launches_per_step=1,
                    config={"workload": f"GEMM {name[5:]} 8192^3, B as [N,K]", "l2": "operands (128-256 MB each) larger than L2"},
                    kind="gemm", replicas_only=True)

    if name == "gemm_f32_exact":
        # the same contraction with DOCC_B200_FLAG_FP32_EXACT: fp32 FMA arithmetic like the reference's loop nest, no tensor cores
        n = 4096
        g.manual_seed(6)
        a = torch.randn(n, n, generator=g).to(dev)
        b = torch.randn(n, n, generator=g).to(dev)
        c = torch.empty(n, n, dtype=torch.float32, device=dev)

        def step():
            ops.gemm(a, b, c, transb=True, flags=ops.FLAG_FP32_EXACT)

        return dict(step=step, units=2 * n ** 3, unit="TFLOP/s", scale=1e-12, metric="gemm_f32_exact_tflops", dtype="f32", bound="fma",
                    peak=148 * 128 * 2 * 1.965e-3, peak_source="of the nominal FFMA rate, 148 SMs x 128 lanes x 2 x 1.965 GHz (no measured figure)",
                    launches_per_step=1, flush=True,
                    config={"workload": "GEMM fp32 4096^3 with FLAG_FP32_EXACT (FFMA kernel), B as [N,K]", "l2": "flushed between steps"},
                    kind="gemm", replicas_only=True)

    # ---- sharded workloads -----------------------------------------------------------------------------
    # `strong`: ONE configuration is split over the ranks by a GatherPlan (chunk-major, rank order inside a chunk); the
    # rank's kernels write straight into its slices of the preallocated gathered buffer and the chunks' all-gathers
    # run in place on a second stream. Otherwise every rank runs the whole configuration on its own (rank-seeded) data.
    def plan_for(total):
        if not strong or world == 1:
            return None
        chunks = GATHER_CHUNKS if total % (world * GATHER_CHUNKS) == 0 else 1
        return GatherPlan(total, rank, world, chunks)

    if name in ("conv_f32", "conv_bf16"):
        n_total = 32
        g.manual_seed(2 if strong else 2 + 1000 * rank)
        x = torch.randn(n_total, 64, 56, 56, generator=g)
        plan = plan_for(n_total)
        if plan:
            x = plan.local_input(x)
        n_local = x.shape[0]
        w = torch.nn.init.kaiming_normal_(torch.empty(128, 64, 3, 3), generator=g)
        bias = torch.zeros(128)
        if name == "conv_bf16":
            x, w = x.bfloat16(), w.bfloat16()
        x, w, bias = x.to(dev), w.to(dev), bias.to(dev)
        y = torch.empty(n_total if plan else n_local, 128, 56, 56, dtype=torch.float32, device=dev)

        def conv_call(xv, yv):  # the C-ABI call a generated host function makes; output buffer owned by the caller
            ops.call("docc_b200_conv", ops._prec(xv), ord("s"), 2, ops._arr(xv.shape), ops._arr((3, 3)), ops._arr((1, 1)),
                     ops._arr((1, 1, 1, 1)), ops._arr((1, 1)), 128, 1, ops._ptr(xv), ops._ptr(w), ops._ptr(bias), ops._ptr(yv), 0)

        flops = 2 * n_local * 128 * 56 * 56 * 64 * 9
        common = dict(units=flops, unit="TFLOP/s", scale=1e-12, metric=name + "_tflops",
                      dtype="bf16" if name == "conv_bf16" else "f32(split-bf16x3)", bound="tensor",
                      peak=peaks["bf16_tflops"] / (1 if name == "conv_bf16" else 3), launches_per_step=None, kind="conv")
        wtext = f"conv2d {name[5:]} [32,64,56,56]*[128,64,3,3] s1 p1 (BASELINE config 3)"
        if plan:
            return dict(step=None, config={"workload": wtext, "batch_per_gpu": n_local, "l2": "flushed between steps"}, flush=True,
                        plan=plan, full_out=y, gather_bytes=y.numel() * 4,
                        chunk=lambda c, out: conv_call(plan.local_chunk(x, c), out), **common)
        # Steps of 25-70 us: an event pair per step (what the L2 flush between steps needs) adds the events' own latency and
        # a 2 us timestamp granularity to every step. Instead the steps run back to back over six input/output sets
        # (64-77 MB each, 385-462 MB in all), so no step finds its input, or room for its output, in the 126 MB L2.
        n_sets = 6
        xs = [x] + [torch.randn_like(x, dtype=torch.float32).to(x.dtype) for _ in range(n_sets - 1)]
        ys = [y] + [torch.empty_like(y) for _ in range(n_sets - 1)]
        cargs = [(ops._prec(xi), ord("s"), 2, ops._arr(xi.shape), ops._arr((3, 3)), ops._arr((1, 1)), ops._arr((1, 1, 1, 1)),
                  ops._arr((1, 1)), 128, 1, ops._ptr(xi), ops._ptr(w), ops._ptr(bias), ops._ptr(yi), 0) for xi, yi in zip(xs, ys)]
        state = {"i": 0}

        def step():
            i = state["i"] % n_sets
            state["i"] += 1
            ops.call("docc_b200_conv", *cargs[i])
            return ys[i]

        return dict(step=step, config={"workload": wtext, "batch_per_gpu": n_local,
                                       "l2": "inputs and outputs rotated over 6 buffer sets, larger than L2"},
                    steps_scale=20, **common)  # 20-60 us steps: twenty times the steps of the other extras cost nothing and
        # keep the first launch's latency and the host's jitter out of the per-step figure

    if name in ("attention", "attention_causal"):
        causal = name.endswith("causal")
        bh_total = 8
        g.manual_seed(3 if strong else 3 + 1000 * rank)
        q, k, v = (torch.randn(bh_total, 16, 2048, 128, generator=g) for _ in range(3))
        plan = plan_for(bh_total)
        if plan:
            q, k, v = (plan.local_input(t_) for t_ in (q, k, v))
        q, k, v = (t_.bfloat16().to(dev) for t_ in (q, k, v))
        b_local = q.shape[0]
        o = torch.empty((bh_total if plan else b_local, 16, 2048, 128), dtype=torch.bfloat16, device=dev)
        null = ops.ctypes.cast(None, ops.ctypes.POINTER(ops.ctypes.c_int64))

        def attn_call(qv, kv, vv, ov):
            ops.call("docc_b200_attention", ord("b"), qv.shape[0], 16, 2048, 2048, 128, 1.0 / 128 ** 0.5, int(causal), ops._ptr(qv), null,
                     ops._ptr(kv), null, ops._ptr(vv), null, ops._ptr(ov), null, 0)

        aargs = (ord("b"), b_local, 16, 2048, 2048, 128, 1.0 / 128 ** 0.5, int(causal), ops._ptr(q), null, ops._ptr(k), null,
                 ops._ptr(v), null, ops._ptr(o), null, 0)

        def step():
            ops.call("docc_b200_attention", *aargs)
            return o

        flops = 4 * b_local * 16 * 2048 * 2048 * 128 // (2 if causal else 1)
        return dict(step=step, units=flops, unit="TFLOP/s", scale=1e-12, metric=name + "_tflops", dtype="bf16",
                    bound="tensor", peak=peaks["bf16_tflops"], launches_per_step=1,
                    config={"workload": f"attention bf16 [8,16,2048,128] causal={causal} (BASELINE config 4)",
                            "batch_per_gpu": b_local,
                            # Q, K, V and O are 67 MB each: one step's operands (268 MB) do not fit the 126 MB L2, so steps run back to back
                            "l2": "flushed between steps" if plan else "operands of a step (268 MB) larger than L2"},
                    flush=bool(plan), kind="attention",
                    plan=plan, full_out=o, gather_bytes=o.numel() * 2,
                    chunk=(lambda c, out: attn_call(plan.local_chunk(q, c), plan.local_chunk(k, c), plan.local_chunk(v, c), out))
                    if plan else None)

    if name in ("block_f32", "block_bf16"):
        bf = name.endswith("bf16")
        b_total = 32
        d, heads, dff, seq = 1024, 16, 4096, 512
        torch.manual_seed(4 if strong else 4 + 1000 * rank)
        p = {"ln1_g": torch.ones(d), "ln1_b": torch.zeros(d), "ln2_g": torch.ones(d), "ln2_b": torch.zeros(d)}
        for nm, shp in (("w_qkv", (3 * d, d)), ("w_o", (d, d)), ("w_1", (dff, d)), ("w_2", (d, dff))):
            p[nm] = torch.nn.init.xavier_uniform_(torch.empty(*shp))
        for nm, n in (("b_qkv", 3 * d), ("b_o", d), ("b_1", dff), ("b_2", d)):
            p[nm] = torch.zeros(n)
        x = torch.randn(b_total, seq, d)
        plan = plan_for(b_total)
        if plan:
            x = plan.local_input(x)
        b_local = x.shape[0]
        small = ("ln1_g", "ln1_b", "ln2_g", "ln2_b", "b_qkv", "b_o", "b_1", "b_2")
        pd = {k_: (v_.to(dev) if (k_ in small or not bf) else v_.bfloat16().to(dev)) for k_, v_ in p.items()}
        x = (x.bfloat16() if bf else x).to(dev)
        y = torch.empty((b_total if plan else b_local, seq, d), dtype=x.dtype, device=dev)
        bp = ops.BlockParams()
        bp.seq, bp.d_model, bp.n_heads, bp.d_ff, bp.eps = seq, d, heads, dff, 1e-5
        for f_ in ops.BLOCK_FIELDS:
            setattr(bp, f_, ops._ptr(pd[f_]).value or 0)

        def block_call(xv, yv):
            bp.batch = xv.shape[0]
            ops.call("docc_b200_transformer_block", ops._prec(xv), ops.ctypes.byref(bp), ops._ptr(xv), ops._ptr(yv), 0)

        def step():
            block_call(x, y)
            return y

        T = b_local * seq
        flops = 2 * T * d * (3 * d + d + 2 * dff) + 4 * b_local * heads * seq * seq * (d // heads)
        return dict(step=step, units=flops, unit="TFLOP/s", scale=1e-12, metric=name + "_tflops",
                    dtype="bf16" if bf else "f32(split-bf16x3)", bound="tensor",
                    peak=peaks["bf16_tflops_sustained"] / (1 if bf else 3), launches_per_step=None,
                    config={"workload": f"pre-LN encoder block {'bf16' if bf else 'fp32'} d1024 h16 ff4096 [32,512,1024] "
                                        "(BASELINE config 5)", "batch_per_gpu": b_local,
                            # a step streams its 33-67 MB input, 25-50 MB of weights and 370-740 MB of intermediates through L2
                            "l2": "flushed between steps" if plan else "working set of a step (over 400 MB) larger than L2"},
                    flush=bool(plan), kind="block", plan=plan, full_out=y, gather_bytes=y.numel() * y.element_size(),
                    chunk=(lambda c, out: block_call(plan.local_chunk(x, c), out)) if plan else None)

    raise SystemExit(f"unknown workload {name}")


def time_workload(wl, torch, dist, ops, steps, warmup, world, rank, sample_clocks=False):
    """Device-timed loop: W warm-ups, then K steps bracketed by barrier + synchronize, max over ranks.
    Returns (ms per step, launches, clocks, compute ms per step): the last is the time of the step's kernels alone
    (same chunks, no gather) when the step ends with a gather (split-and-gather mode), else None."""
    dev_index = torch.cuda.current_device()
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if wl.get("flush") else None
    plan = wl.get("plan")
    comm = torch.cuda.Stream() if plan else None

    def full_step():
        if plan is None:
            wl["step"]()
            return
        # kernels of chunk c on the current stream, its in-place all-gather on the second stream behind an event
        plan.run(wl["full_out"], wl["chunk"], comm_stream=comm)
        torch.cuda.current_stream().wait_stream(comm)  # the step ends when the gathered buffer is complete

    def compute_only():
        for c in range(plan.chunks):
            wl["chunk"](c, plan.out_slice(wl["full_out"], c))

    for _ in range(max(warmup, 3)):
        full_step()
    torch.cuda.synchronize()
    one_step, comp_step = full_step, (compute_only if plan else None)
    sampler = ClockSampler(dev_index) if sample_clocks else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    ops.launch_count(reset=True)

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if flush_buf is None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                fn()
            end.record()
            torch.cuda.synchronize()
            return start.elapsed_time(end) / steps
        # L2 flush between steps: time each step with its own event pair so the flush is not counted
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for s, e in evs:
            flush_buf.fill_(1)
            s.record()
            fn()
            e.record()
        torch.cuda.synchronize()
        return sum(s.elapsed_time(e) for s, e in evs) / steps

    ms = timed(one_step)
    launches = ops.launch_count()
    compute_ms = timed(comp_step) if plan is not None else None
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms, compute_ms if compute_ms is not None else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0].item())
        if compute_ms is not None:
            compute_ms = float(t[1].item())
    return ms, launches, clocks, compute_ms


def e2e_softmax(torch, dist, ops, steps, warmup, world):
    """Same metric through the C ABI with HOST buffers: pinned input -> H2D -> kernel -> D2H inside the timed region."""
    rows, cols = 8192, 4096
    x = (3 * torch.randn(rows, cols)).pin_memory()
    y = torch.empty(rows, cols).pin_memory()
    shape, axes = ops._arr((rows, cols)), ops._arr((1,))

    def step():
        ops.call("docc_b200_softmax", ord("s"), 2, shape, 1, axes, x.data_ptr(), y.data_ptr(), ops.FLAG_HOST_PTRS)

    for _ in range(max(warmup, 3)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert abs(float(y[0].sum()) - 1.0) < 1e-3  # device -> host read of the step's result
    return {"value": world * 2 * rows * cols * 4 / (ms * 1e-3) * 1e-9, "unit": "GB/s", "ms_per_step": ms,
            "h2d_bytes_per_step": rows * cols * 4, "d2h_bytes_per_step": rows * cols * 4,
            "path": "docc_b200_softmax(DOCC_B200_FLAG_HOST_PTRS) on pinned host buffers, chunked H2D/kernel/D2H pipeline"}


def _all_cores(oracle):
    # all the host cores this process may use, whatever OMP_NUM_THREADS the launcher exported (torchrun sets 1)
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    oracle.set_num_threads(n)
    return n


def cpu_softmax_baseline(budget_s=12.0, max_reps=20):
    """Times the oracle (the reference's 7-loop-nest expansion, OpenMP on the outermost maps) on the full config."""
    import oracle

    _all_cores(oracle)
    rows, cols = 8192, 4096
    x = (3 * np.random.RandomState(1).randn(rows, cols)).astype(np.float32)
    oracle.softmax(x[:256], [1])
    times = []
    t_all = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_all) < budget_s:
        t0 = time.perf_counter()
        oracle.softmax(x, [1])
        times.append(time.perf_counter() - t0)
    best = float(np.median(times))
    return {"value": 2 * rows * cols * 4 / best * 1e-9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"full [8192,4096] fp32 tensor, median of {len(times)} runs ({best * 1e3:.1f} ms each)",
            "ms_per_step": best * 1e3}


def cpu_extra_baseline(name):
    """CPU baseline of an extra workload on a bounded sample (a few seconds): the oracle's restatement of the node, or, for
    config 1, the BLAS dgemm the reference itself calls on the CPU (gemm_node.cpp:449-509; numpy's OpenBLAS stands in for
    the unpinned -lblas). Returned in the workload's unit, scaled from the sample by the work it contains."""
    import oracle
    import torch

    cores = _all_cores(oracle)

    def timed(fn, reps=3):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return float(np.median(ts))

    if name == "gemm_f64":
        rs = np.random.RandomState(0)
        a, b = rs.rand(1000, 1000), rs.rand(1000, 1000)
        torch.set_num_threads(cores)
        t = timed(lambda: a @ b, 10)
        return {"value": 2e9 / t * 1e-12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                "sample": f"full 1000^3 problem through OpenBLAS dgemm (numpy), median of 10 ({t * 1e3:.2f} ms)"}
    if name.startswith("conv"):
        rs = np.random.RandomState(2)
        x = rs.randn(2, 64, 56, 56).astype(np.float32)
        w = (rs.randn(128, 64, 3, 3) * (2.0 / 576) ** 0.5).astype(np.float32)
        t = timed(lambda: oracle.conv(x, w, np.zeros(128, dtype=np.float32), pads=[1, 1, 1, 1]), 2)
        return {"value": 2 * 2 * 128 * 56 * 56 * 576 / t * 1e-12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                "sample": f"2 of the 32 images, fp32 oracle loop nest ({t * 1e3:.0f} ms)"}
    if name.startswith("attention"):
        rs = np.random.RandomState(3)
        causal = name.endswith("causal")
        q, k, v = (rs.randn(1, 2, 2048, 128).astype(np.float32) for _ in range(3))
        t = timed(lambda: oracle.attention(q, k, v, causal=causal), 2)
        fl = 4 * 2 * 2048 * 2048 * 128 / (2 if causal else 1)
        return {"value": fl / t * 1e-12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                "sample": f"2 of the 128 (batch, head) problems, fp32 oracle composition ({t * 1e3:.0f} ms)"}
    if name.startswith("block"):
        d, dff, heads, seq = 1024, 4096, 16, 512
        rs = np.random.RandomState(4)
        p = {"ln1_g": np.ones(d, np.float32), "ln1_b": np.zeros(d, np.float32), "ln2_g": np.ones(d, np.float32), "ln2_b": np.zeros(d, np.float32)}
        for nm, shp in (("w_qkv", (3 * d, d)), ("w_o", (d, d)), ("w_1", (dff, d)), ("w_2", (d, dff))):
            p[nm] = (rs.rand(*shp).astype(np.float32) - 0.5) * 2 * (6.0 / sum(shp)) ** 0.5
        for nm, n in (("b_qkv", 3 * d), ("b_o", d), ("b_1", dff), ("b_2", d)):
            p[nm] = np.zeros(n, np.float32)
        x = rs.randn(1, seq, d).astype(np.float32)
        t = timed(lambda: oracle.transformer_block(x, p, heads), 2)
        fl = 2 * seq * d * (3 * d + d + 2 * dff) + 4 * heads * seq * seq * (d // heads)
        return {"value": fl / t * 1e-12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                "sample": f"1 of the 32 sequences, fp32 oracle composition ({t * 1e3:.0f} ms)"}
    return None


def e2e_extra(name, torch, ops, steps=5):
    """The workload through the C ABI with HOST buffers (pinned): H2D of the inputs, the kernels and D2H of the result are
    inside the timed region, as generated host code with the "WithTransfers" dispatchers does it."""
    pin = lambda t_: t_.contiguous().pin_memory()
    if name == "gemm_f64":
        rs = np.random.RandomState(0)
        a, b = pin(torch.from_numpy(rs.rand(1000, 1000))), pin(torch.from_numpy(rs.rand(1000, 1000)))
        c = pin(torch.empty(1000, 1000, dtype=torch.float64))
        one, zero = ops.ctypes.c_double(1.0), ops.ctypes.c_double(0.0)
        vp = ops.ctypes.c_void_p

        def call():
            ops.call("docc_b200_gemm", ord("d"), 101, 111, 111, 1000, 1000, 1000, ops.ctypes.cast(ops.ctypes.pointer(one), vp), vp(a.data_ptr()), 1000,
                     vp(b.data_ptr()), 1000, ops.ctypes.cast(ops.ctypes.pointer(zero), vp), vp(c.data_ptr()), 1000, ops.FLAG_HOST_PTRS)

        units, h2d, d2h = 2e9, 16e6, 8e6
    elif name in ("conv_f32", "conv_bf16"):
        g = torch.Generator().manual_seed(2)
        x = torch.randn(32, 64, 56, 56, generator=g)
        w = torch.nn.init.kaiming_normal_(torch.empty(128, 64, 3, 3), generator=g)
        if name == "conv_bf16":
            x, w = x.bfloat16(), w.bfloat16()
        x, w, bias = pin(x), pin(w), pin(torch.zeros(128))
        y = pin(torch.empty(32, 128, 56, 56))
        vp = ops.ctypes.c_void_p

        def call():
            ops.call("docc_b200_conv", ops._prec(x), ord("s"), 2, ops._arr(x.shape), ops._arr((3, 3)), ops._arr((1, 1)), ops._arr((1, 1, 1, 1)),
                     ops._arr((1, 1)), 128, 1, vp(x.data_ptr()), vp(w.data_ptr()), vp(bias.data_ptr()), vp(y.data_ptr()), ops.FLAG_HOST_PTRS)

        units = 2 * 32 * 128 * 56 * 56 * 576
        h2d, d2h = x.numel() * x.element_size() + w.numel() * w.element_size() + 512, y.numel() * 4
    else:
        return None
    for _ in range(2):
        call()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        call()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    return {"value": units / (ms * 1e-3) * 1e-12, "unit": "TFLOP/s", "ms_per_step": ms, "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "path": "C ABI with DOCC_B200_FLAG_HOST_PTRS on pinned host buffers"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_softmax_baseline(budget_s=20.0, max_reps=max(args.steps + args.warmup, 3))
    line = {"impl": "reference", "metric": "softmax_hbm_gbs", "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": headline_config(),
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of docc's SoftmaxNode expansion (7 loop nests, 6 temporaries), OpenMP on the outermost "
                    "map as docc's openmp target schedules it; the reference itself cannot be built without clang/MLIR/symengine"}
    print(json.dumps(line))


def main():
    global STRONG, GATHER_CHUNKS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="softmax")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--strong", action="store_true",
                    help="headline the split-and-gather reading of a sharded workload (one configuration split over the GPUs)")
    ap.add_argument("--kernel-only", action="store_true", help="skip the e2e and CPU-baseline legs (profiling runs)")
    ap.add_argument("--extra-steps", type=int, default=10)
    ap.add_argument("--gather-chunks", type=int, default=GATHER_CHUNKS, help="chunks per step in the split-and-gather mode")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference(args)
        return
    STRONG = bool(args.strong)
    GATHER_CHUNKS = max(1, int(args.gather_chunks))

    import torch
    import torch.distributed as dist

    from docc_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    numa = bind_near_gpu(local_rank) if world > 1 else {"bound": False, "note": "single rank: left unbound"}
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ops.init(local_rank)
    ops.set_stream(torch.cuda.current_stream().cuda_stream)

    wl = make_workload(args.workload, torch, ops, rank, world, strong=STRONG)
    ms, launches, clocks, compute_ms = time_workload(wl, torch, dist, ops, args.steps, args.warmup, world, rank, sample_clocks=True)
    peaks = measured_peaks()
    per_gpu = wl["units"] / (ms * 1e-3) * wl["scale"]
    value = per_gpu * (1 if wl.get("replicas_only") else world)
    roof = {"bound": wl["bound"], "achieved": per_gpu, "peak": wl["peak"], "unit": wl["unit"],
            "frac": (per_gpu / wl["peak"]) if wl["peak"] else None, "traffic": None,
            "peak_source": wl.get("peak_source", f"of {peaks['source']}")}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload)

    split = bool(wl.get("plan"))
    line = {"metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "replicas" if wl.get("replicas_only") else ("strong" if split else "weak"), "vs_baseline": None, "dtype": wl["dtype"],
            "data": "synthetic", "config": wl["config"], "roofline": roof, "gpu_launches": int(launches), "clocks": clocks}
    if split:
        line["compute_ms"] = compute_ms
        line["gather_exposed_ms"] = ms - compute_ms if compute_ms is not None else None

    if args.workload == "softmax" and not args.kernel_only:
        line["e2e"] = e2e_softmax(torch, dist, ops, max(args.steps // 5, 5), args.warmup, world)
        line["e2e"]["host_binding_rank0"] = numa
        if rank == 0 and world == 1:
            line["cpu_baseline"] = {k: v for k, v in cpu_softmax_baseline().items() if k != "ms_per_step"}

    if not args.no_extras and args.workload == "softmax":
        extras = []
        names = ["gemm_f64", "gemm_bf16", "gemm_f32", "gemm_f32_exact", "conv_f32", "conv_bf16", "attention", "attention_causal", "block_f32", "block_bf16"]
        for nm in names:
            try:
                w2 = make_workload(nm, torch, ops, rank, world)
                ms2, l2, clk2, _ = time_workload(w2, torch, dist, ops, args.extra_steps * w2.get("steps_scale", 1), 3, world, rank,
                                                 sample_clocks=(rank == 0))
                pg = w2["units"] / (ms2 * 1e-3) * w2["scale"]
                ex = {"metric": w2["metric"], "value": pg * (1 if w2.get("replicas_only") else world),
                      "unit": w2["unit"], "ms_per_step": ms2, "steps": args.extra_steps * w2.get("steps_scale", 1), "dtype": w2["dtype"],
                      "config": w2["config"],
                      "roofline": {"bound": w2["bound"], "achieved": pg, "peak": w2["peak"],
                                   "frac": (pg / w2["peak"]) if w2["peak"] else None, "unit": w2["unit"],
                                   "traffic": NCU_TRAFFIC_BYTES.get(nm),
                                   "peak_source": w2.get("peak_source", f"of {peaks['source']}")},
                      "gpu_launches": int(l2), "clocks": clk2}
                del w2
                torch.cuda.empty_cache()
                if world == 1 and not args.kernel_only:
                    e2e = e2e_extra(nm, torch, ops)
                    if e2e:
                        ex["e2e"] = e2e
                    cb = cpu_extra_baseline(nm)
                    if cb:
                        ex["cpu_baseline"] = cb
                # the split-and-gather reading of the sharded configurations, next to the weak one
                if world > 1 and nm not in ("gemm_f64", "gemm_bf16", "gemm_f32", "gemm_f32_exact"):
                    w3 = make_workload(nm, torch, ops, rank, world, strong=True)
                    ms3, _, _, comp3 = time_workload(w3, torch, dist, ops, args.extra_steps, 3, world, rank)
                    ex["split_gather"] = {
                        "ms_per_step": ms3, "compute_ms": comp3, "gather_exposed_ms": ms3 - comp3 if comp3 is not None else None,
                        "speedup_vs_one_gpu": ms2 / ms3, "chunks": w3["plan"].chunks,
                        "gathered_bytes_per_rank": int(w3["gather_bytes"] * (world - 1) // world),
                        "nvlink_bound_ms": w3["gather_bytes"] * (world - 1) / world / 770e9 * 1e3,
                        "note": "one configuration split over the GPUs; in-place NCCL all-gather per chunk on a second stream; compute_ms = "
                                "the same chunks' kernels alone (launches issued one by one: short steps are paced by the host); "
                                "speed-up against the same configuration on one GPU of this run (the weak reading above); "
                                "NVLink bound = bytes a rank receives / 770 GB/s measured peer copy rate"}
                    del w3
                    torch.cuda.empty_cache()
                extras.append(ex)
            except Exception as exc:  # an extra must never take the headline line down
                extras.append({"metric": nm, "error": f"{type(exc).__name__}: {exc}"[:300]})
        line["extras"] = extras

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()

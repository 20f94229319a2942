#!/usr/bin/env python
"""Benchmark of the tensor-operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One STEP is one pass of the sharded large-tensor chain of the baseline configuration:
broadcast Mul  A[8,1,2048,2048] x B[1,16,1,2048] -> O[8,16,2048,2048] (2 GiB), then a full-tensor
ReduceSum and a full-tensor ReduceMax of O.  With N ranks (one process per GPU, torchrun) the
tensor is split on dim 0 (STRONG scaling: the total work is the fixed 2 GiB tensor), B is
replicated, and the per-rank double partials of both reductions travel in one NCCL all-gather of
16 bytes per rank (the C entry points of libsb200_nccl.so) and are folded in rank order on every rank.  Inputs are seeded synthetic tensors (U(-1,1) and N(0,1)) resident in HBM before the
timed region; every step touches > 2 GiB per GPU at N=1 (> 256 MiB at N=8), larger than the
126 MB L2, so no L2 flush is interposed.

Reported on one JSON line: the whole-job effective HBM GB/s (algorithmic bytes of the step /
max-over-ranks device time), the roofline of the dominant kernel (the broadcast Mul) measured
live with CUDA events, the same metric end to end through the Shadow Network API with host
buffers (e2e), a per-operator sweep at >= 256 MB sizes, and the reference's CPU implementation
timed on the host cores (cpu_baseline).  `--impl reference` times only that CPU implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC, UNIT = "effective_hbm_gb_per_s", "GB/s"
NOMINAL_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0
A_SHAPE, B_SHAPE, O_SHAPE = (8, 1, 2048, 2048), (1, 16, 1, 2048), (8, 16, 2048, 2048)
SEED_A, SEED_B = 20240650, 20240651
MUL, RED_SUM, RED_MAX = 2, 1, 2


def numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def step_bytes(a_shape, b_shape, o_shape):
    """Algorithmic bytes: every input read once, every output written once, 4 B per element."""
    mul = 4 * (numel(a_shape) + numel(b_shape) + numel(o_shape))
    red = 4 * (numel(o_shape) + 1)
    return {"binary_broadcast_mul": mul, "reduce_sum_all": red, "reduce_max_all": red}


def make_inputs(a_shape, b_shape):
    a = np.random.Generator(np.random.PCG64(SEED_A)).uniform(-1.0, 1.0, size=a_shape).astype(np.float32)
    b = np.random.Generator(np.random.PCG64(SEED_B)).normal(0.0, 1.0, size=b_shape).astype(np.float32)
    return a, b


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


def ncu_traffic():
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get("bcast_reuse_kernel_c5_bytes_per_launch")
    except Exception:
        return None


class ClockSampler:
    """SM clock and throttle reasons of one GPU while work runs, read by an `nvidia-smi -lms`
    child process.  (Polling NVML from a thread of this process takes driver locks that the
    launches of a short timed region then wait for: at 8 GPUs it doubled the step time.)"""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int, period_ms: int = 20, ready_wait_s: float = 15.0):
        self.index, self.period_ms, self.ready_wait_s = index, period_ms, ready_wait_s
        self.proc, self.samples, self.reasons, self.max_mhz = None, [], set(), None

    def __enter__(self):
        import subprocess
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
        # wait for the child's first line: with eight of them starting at once on an 8-GPU box a child needs
        # longer to come up than a short timed region lasts, and the region would go unsampled
        self.first = ""
        if self.proc is not None and self.ready_wait_s > 0:
            import select
            try:
                ready, _, _ = select.select([self.proc.stdout], [], [], self.ready_wait_s)
                if ready:
                    self.first = self.proc.stdout.readline()
            except Exception:
                pass
        return self

    def __exit__(self, *exc):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            out = self.proc.stdout.read()      # through the same reader as the first line: nothing buffered is lost
        except Exception:
            out = ""
        # (the first line was taken before the barrier, with the GPU idle: it only shows that the child is up)
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append(int(float(parts[0])))
                self.max_mhz = int(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[2:6]):
                if val.lower().startswith("active"):
                    self.reasons.add(name)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------------------
# reference CPU implementation (oracle/_ref, else the C port) on a bounded sample
# --------------------------------------------------------------------------------------------------
SAMPLE_A, SAMPLE_B, SAMPLE_O = (1, 1, 512, 2048), (1, 16, 1, 2048), (1, 16, 512, 2048)
SAMPLE_TEXT = "dim-0 slice 1 of 8 and rows 0..511 of 2048 of the workload: A[1,1,512,2048] x B[1,16,1,2048] " \
              "-> [1,16,512,2048] (1/32 of the step), then full ReduceSum and ReduceMax"


class CpuChain:
    """The step's three operators on the sample, through the reference's Network API."""

    def __init__(self):
        from oracle import oracle as orc
        self.orc = orc
        self.lib = orc.ref_library()
        self.kind = "reference" if self.lib is not None else "port"
        self.net = None

    def prepare(self, a, b):
        self.a, self.b = a, b
        if self.lib is not None:
            from shadow_b200.netapi import Net
            net = Net(self.lib, "c5_sample").input({"a": a.shape, "b": b.shape})
            net.op("Binary", ["a", "b"], ["o"], operation=MUL)
            net.op("Reduce", ["o"], ["s"], operation=RED_SUM, axes=[], keep_dims=False)
            net.op("Reduce", ["o"], ["m"], operation=RED_MAX, axes=[], keep_dims=False)
            net.load("Native", out_blobs=["s", "m"])
            net.forward({"a": a, "b": b})   # first call: the reference builds its index tables here
            self.net = net

    def run(self):
        if self.net is not None:
            self.net.forward()              # operators only: inputs are already in the blobs
            return float(self.net.blob("s").ravel()[0]), float(self.net.blob("m").ravel()[0])
        o = self.orc.binary(self.a, self.b, MUL)
        return (float(self.orc.reduce(o, RED_SUM, [], False).ravel()[0]),
                float(self.orc.reduce(o, RED_MAX, [], False).ravel()[0]))


N_SLICES = (A_SHAPE[0]) * (A_SHAPE[2] // SAMPLE_A[2])   # 32 slices of 1/32 make up the whole step


def time_cpu(threads: int, steps: int, warmup: int, slices: int = N_SLICES):
    """The chain on `slices` of the 32 dim-0 x row slices of the workload (32 = the whole step), spread
    over `threads` host threads (the reference path itself is single-threaded): thread t runs slices
    t, t + threads, ... one after the other, each through its own reference Network.  Returns
    (GB/s, ms per step, kind, (sum, max) over the slices, slice 0 of A)."""
    a_full, b = make_inputs(A_SHAPE, B_SHAPE)
    rows = SAMPLE_A[2]
    chains = []
    for t in range(slices):
        n, r0 = t % A_SHAPE[0], (t // A_SHAPE[0]) * rows
        a = np.ascontiguousarray(a_full[n:n + 1, :, r0:r0 + rows, :])
        chains.append((CpuChain(), a))
    del a_full
    threads = max(1, min(threads, slices))

    def on_threads(fn):
        def work(t):
            for i in range(t, slices, threads):
                fn(i)
        ws = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
        [w.start() for w in ws]
        [w.join() for w in ws]

    on_threads(lambda i: chains[i][0].prepare(chains[i][1], b))
    results = [None] * slices

    def run_one(i):
        results[i] = chains[i][0].run()

    for _ in range(warmup):
        on_threads(run_one)
    t0 = time.perf_counter()
    for _ in range(steps):
        on_threads(run_one)
    dt = time.perf_counter() - t0
    nbytes = sum(step_bytes(SAMPLE_A, SAMPLE_B, SAMPLE_O).values()) * slices
    # the slices' float sums added in double in slice order; the maximum is exact
    total = (float(np.sum(np.array([r[0] for r in results], dtype=np.float64))), max(r[1] for r in results))
    return nbytes * steps / dt / 1e9, dt / steps * 1e3, chains[0][0].kind, total, chains[0][1], results[0]


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = max(1, min(os.cpu_count() or 1, N_SLICES))
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 1))
    gbs, ms, kind, total, _, _ = time_cpu(threads, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C5 chain: broadcast Mul A[8,1,2048,2048]xB[1,16,1,2048] -> [8,16,2048,2048] (2 GiB), "
                               "ReduceSum all axes, ReduceMax all axes, on the host cores",
                   "how": "the whole step, cut into %d slices (%s) that %d host threads work through, each slice "
                          "through the reference's own Network API" % (N_SLICES, SAMPLE_TEXT, threads),
                   "bytes_per_step": sum(step_bytes(A_SHAPE, B_SHAPE, O_SHAPE).values())},
        "cpu_baseline": {"value": round(gbs, 4), "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": "the full step: %d slices, each %s" % (N_SLICES, SAMPLE_TEXT)},
        "e2e": {"value": round(gbs, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "results": {"sum": total[0], "max": total[1]},
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------------------
# B200 arm
# --------------------------------------------------------------------------------------------------
def per_op_sweep(torch, F, device, peak):
    """Every operator family at a tensor size >= 256 MB (the roofline claim), L2-cold by size."""
    def t(shape, lo=-1.0, hi=1.0):
        return torch.empty(shape, device=device).uniform_(lo, hi)

    rows = []

    def bench(name, fn, nbytes, iters=10):
        """Times ONE call of `fn` per sample.  The call is captured in a CUDA graph and the graph is
        replayed between two events, so the host cost of the Python/ctypes call (about as long as
        the shorter kernels here) stays out of the measurement."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in evs:
            a.record()
            graph.replay()
            b.record()
        torch.cuda.synchronize()
        ms = statistics.median(a.elapsed_time(b) for a, b in evs)
        gbs = nbytes / ms / 1e6
        rows.append({"op": name, "bytes": nbytes, "ms": round(ms, 4), "gb_per_s": round(gbs, 1),
                     "frac_of_8tbs": round(gbs / NOMINAL_PEAK_GBS, 4), "frac_of_measured": round(gbs / peak, 4)})
        del graph

    c1 = (512, 64, 56, 56)
    a, c, y = t(c1), t(c1), torch.empty(c1, device=device)
    b = torch.randn(1, 64, 1, 1, device=device)
    n = a.numel()
    for name, code in (("Add", 0), ("Mul", 2), ("Max", 5)):
        bench("binary_broadcast_%s[512,64,56,56]+[1,64,1,1]" % name, lambda: F.binary(a, b, code, out=y), 8 * n + 256)
    bench("binary_same_Add[512,64,56,56]", lambda: F.binary(a, c, 0, out=y), 12 * n)
    bench("binary_scalar_Mul[512,64,56,56]", lambda: F.binary_scalar(a, 1.5, 2, out=y), 8 * n)
    a.uniform_(0.5, 2.0)
    c.uniform_(0.5, 2.0)
    bench("binary_same_Div[512,64,56,56]", lambda: F.binary(a, c, 3, out=y), 12 * n)
    bench("binary_same_Pow[512,64,56,56]", lambda: F.binary(a, c, 4, out=y), 12 * n)
    a.uniform_(-1.0, 1.0)
    c.uniform_(-1.0, 1.0)
    bench("eltwise_Sum_3_inputs[512,64,56,56]", lambda: F.eltwise([a, c, a], 1, [0.5, 0.25, 2.0], out=y), 16 * n)
    bench("eltwise_Max_2_inputs[512,64,56,56]", lambda: F.eltwise([a, c], 2, out=y), 12 * n)
    alpha = torch.randn(512, 64, device=device)
    bench("axpy[512,64,56,56]", lambda: F.axpy(alpha, a, c, out=y), 12 * n + 4 * 512 * 64)
    del a, c, y
    c2 = (512, 256, 28, 28)
    x, y = torch.empty(c2, device=device).normal_(0, 2), torch.empty(c2, device=device)
    n = x.numel()
    for name, code in (("Relu", 1), ("Leaky", 2), ("Sigmoid", 3), ("SoftPlus", 4), ("Tanh", 5), ("Relu6", 6), ("HardSwish", 7),
                       ("Gelu", 8)):
        bench("activate_%s[512,256,28,28]" % name, lambda: F.activate(x, code, 0.1, out=y), 8 * n)
    slopes = torch.rand(256, device=device) * 0.3
    bench("activate_PRelu[512,256,28,28]", lambda: F.activate(x, 0, 0.1, slopes, out=y), 8 * n + 4 * 256)
    x.uniform_(-10, 10)
    bench("unary_Exp[512,256,28,28]", lambda: F.unary(x, 4, out=y), 8 * n)
    for name, code in (("Abs", 0), ("Sin", 5), ("Cos", 6), ("Tan", 7), ("Atan", 10), ("Floor", 11), ("Reciprocal", 14)):
        bench("unary_%s[512,256,28,28]" % name, lambda: F.unary(x, code, out=y), 8 * n)
    x.uniform_(-1, 1)
    for name, code in (("Asin", 8), ("Acos", 9)):
        bench("unary_%s[512,256,28,28]" % name, lambda: F.unary(x, code, out=y), 8 * n)
    x.uniform_(0.01, 10)
    bench("unary_Log[512,256,28,28]", lambda: F.unary(x, 3, out=y), 8 * n)
    bench("unary_Sqrt[512,256,28,28]", lambda: F.unary(x, 2, out=y), 8 * n)
    g, bt = torch.randn(256, device=device) * 0.1 + 1, torch.randn(256, device=device) * 0.1
    bench("scale[512,256,28,28]", lambda: F.scale(x, 1, g, bt, out=y), 8 * n + 8 * 256)
    del x, y
    c3 = (1024, 512, 14, 14)
    x = torch.randn(c3, device=device)
    n = x.numel()
    for axes, outs in (((2, 3), 1024 * 512), ((1,), 1024 * 196), ((0, 2, 3), 512)):
        r = torch.empty(outs, device=device)
        for name, code in (("Sum", 1), ("Avg", 4), ("Max", 2), ("Min", 3)):
            bench("reduce_%s%s[1024,512,14,14]" % (name, list(axes)), lambda: F.reduce(x, code, axes, out=r), 4 * (n + outs))
    r = torch.empty(1024 * 512, device=device)
    for name, code in (("L1", 5), ("L2", 6)):
        bench("reduce_%s[2, 3][1024,512,14,14]" % name, lambda: F.reduce(x, code, (2, 3), out=r), 4 * (n + 1024 * 512))
    x.uniform_(0.99, 1.01)
    bench("reduce_Prod[2, 3][1024,512,14,14]", lambda: F.reduce(x, 0, (2, 3), out=r), 4 * (n + 1024 * 512))
    del x
    x, y = torch.empty(16384, 4096, device=device).normal_(0, 3), torch.empty(16384, 4096, device=device)
    bench("softmax_rows[16384,4096]", lambda: F.softmax(x, -1, out=y), 8 * x.numel())
    del x, y
    x, y = torch.randn(1536, 1000, 7, 7, device=device), torch.empty(1536, 1000, 7, 7, device=device)
    bench("softmax_strided_axis1[1536,1000,7,7]", lambda: F.softmax(x, 1, out=y), 8 * x.numel())
    del x, y
    x, y = torch.randn(64, 21, 512, 512, device=device), torch.empty(64, 21, 512, 512, device=device)
    bench("softmax_strided_axis1[64,21,512,512]", lambda: F.softmax(x, 1, out=y), 8 * x.numel())
    del x, y
    x, y = torch.randn(128, 512, 38, 38, device=device), torch.empty(128, 512, 38, 38, device=device)
    bench("normalize_l2_axis1[128,512,38,38]", lambda: F.normalize(x, 1, 2.0, 1e-12, out=y), 8 * x.numel())
    del x, y
    x, y = torch.randn(131072, 512, device=device), torch.empty(131072, 512, device=device)
    bench("normalize_l2_rows[131072,512]", lambda: F.normalize(x, 1, 2.0, 1e-12, out=y), 8 * x.numel())
    del x, y
    x, y = torch.randn(512, 64, 56, 56, device=device), torch.empty(512, 64, 56, 56, device=device)
    mean, var = torch.randn(64, device=device), torch.rand(64, device=device) + 0.1
    bench("batch_norm[512,64,56,56]", lambda: F.batch_norm(x, mean, var, 1.0, 1e-5, out=y), 8 * x.numel() + 8 * 64)
    gs, gb = torch.randn(64, device=device), torch.randn(64, device=device)
    bench("group_norm_g8_affine[512,64,56,56]", lambda: F.group_norm(x, 8, gs, gb, 1e-5, out=y), 8 * x.numel() + 8 * 64)
    bench("instance_norm[512,64,56,56]", lambda: F.instance_norm(x, None, None, 1e-5, out=y), 8 * x.numel())
    del x, y
    x, y = torch.randn(32768, 4096, device=device), torch.empty(32768, 4096, device=device)
    ls, lb = torch.randn(4096, device=device), torch.randn(4096, device=device)
    bench("layer_norm_affine[32768,4096]", lambda: F.layer_norm(x, [4096], ls, lb, 1e-5, out=y), 8 * x.numel() + 8 * 4096)
    del x, y
    x, y = torch.randn(128, 512, 38, 38, device=device), torch.empty(128, 512, 38, 38, device=device)
    sc = torch.full((512,), 20.0, device=device)
    bench("ssd_normalize_per_position[128,512,38,38]", lambda: F.ssd_normalize(x, sc, False, False, 1e-10, out=y),
          8 * x.numel() + 4 * 512)
    del x, y
    x = torch.randn(128, 256, 56, 56, device=device)
    y = torch.empty(128, 56, 56, 256, device=device)
    bench("permute_nchw_to_nhwc[128,256,56,56]", lambda: F.permute(x, [0, 2, 3, 1], out=y), 8 * x.numel())
    y2 = torch.empty(56, 128, 56, 256, device=device)
    bench("permute_general_2031[128,256,56,56]", lambda: F.permute(x, [2, 0, 3, 1], out=y2), 8 * x.numel())
    del x, y, y2
    a, b = torch.randn(256, 64, 56, 56, device=device), torch.randn(256, 96, 56, 56, device=device)
    y = torch.empty(256, 160, 56, 56, device=device)
    bench("concat_axis1[256,64+96,56,56]", lambda: F.concat([a, b], 1, out=y), 8 * y.numel())
    del a, b
    yp = torch.empty(256, 160, 58, 58, device=device)
    bench("pad_1_1_1_1[256,160,56,56]", lambda: F.pad(y, [1, 1, 1, 1], 0.0, out=yp), 4 * (y.numel() + yp.numel()))
    del yp
    idx = torch.arange(0, 160, 2, device=device, dtype=torch.int32)
    yg = torch.empty(256, 80, 56, 56, device=device)
    bench("gather_axis1_every_2nd[256,160,56,56]", lambda: F.gather(y, idx, 1, out=yg), 8 * yg.numel())
    del yg
    idx = torch.randperm(160, device=device).to(torch.int32)
    yg = torch.empty(256, 160, 56, 56, device=device)
    bench("gather_axis1_permuted[256,160,56,56]", lambda: F.gather(y, idx, 1, out=yg), 8 * yg.numel())
    del y, yg
    x = torch.randn(256, 64, 112, 112, device=device)
    y = torch.empty(256, 64, 56, 56, device=device)
    bench("pooling_max_k2_s2[256,64,112,112]", lambda: F.pooling(x, 0, [2], [2], [0], out=y), 4 * (x.numel() + y.numel()))
    bench("pooling_max_k3_s2_p1[256,64,112,112]", lambda: F.pooling(x, 0, [3], [2], [1], full_pooling=False, out=y),
          4 * (x.numel() + y.numel()))
    bench("pooling_avg_k2_s2[256,64,112,112]", lambda: F.pooling(x, 1, [2], [2], [0], out=y), 4 * (x.numel() + y.numel()))
    del x, y
    x = torch.randn(1024, 2048, 7, 7, device=device)
    y = torch.empty(1024, 2048, 1, 1, device=device)
    bench("pooling_avg_global[1024,2048,7,7]", lambda: F.pooling(x, 1, global_pooling=True, out=y), 4 * (x.numel() + y.numel()))
    return rows


class _DevScalar:
    """A float32 scalar that lives in a Network blob, exposed to torch without a copy."""

    def __init__(self, ptr: int):
        self.__cuda_array_interface__ = {"shape": (1,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def run_e2e(n_local, local_rank, a_host, b_host, steps, warmup, comm, torch):
    """The chain through the Shadow Network API (C++ host library) with HOST buffers: every step's
    Forward copies the pinned inputs to the device and runs Binary/Reduce/Reduce, and the step's two
    results are read back to the host.  Two Networks (each with its own stream, as in the reference:
    one Workspace + Context + stream per Network) are driven by two host threads and take the steps
    alternately, so the input copy of step i+1 runs beside the kernels of step i.  With several
    ranks the step also holds the exchange: each rank's two scalars go through ONE all-gather of
    the C entry points (issued by the main thread in step order) and one 16*N-byte read."""
    import concurrent.futures as cf
    import shadow_b200
    from shadow_b200.netapi import Net
    lib = shadow_b200.host_library()
    a_shape = (n_local,) + A_SHAPE[1:]
    ins = {"a": a_host.data_ptr(), "b": b_host.data_ptr()}
    world = comm.n_ranks if comm is not None else 1
    device = torch.device("cuda", local_rank)

    def make():
        net = Net(lib, "c5").input({"a": a_shape, "b": B_SHAPE})
        net.op("Binary", ["a", "b"], ["o"], operation=MUL)
        net.op("Reduce", ["o"], ["s"], operation=RED_SUM, axes=[], keep_dims=False)
        net.op("Reduce", ["o"], ["m"], operation=RED_MAX, axes=[], keep_dims=False)
        net.load("Native", device_id=local_rank, out_blobs=["s", "m"])
        net.forward(ins)
        return net

    nets = [make(), make()]
    views = None
    if world > 1:
        views = [(torch.as_tensor(_DevScalar(n.device_ptr("s")), device=device),
                  torch.as_tensor(_DevScalar(n.device_ptr("m")), device=device)) for n in nets]
        record = torch.empty(2, dtype=torch.float64, device=device)
        gathered = torch.empty(2 * world, dtype=torch.float64, device=device)
        landing = torch.empty(2 * world, dtype=torch.float64).pin_memory()

    def forward(k):
        torch.cuda.set_device(local_rank)
        nets[k].forward(ins)        # H2D of both inputs, three operators, synchronise

    def results(k):
        if world == 1:
            return float(nets[k].blob("s").ravel()[0]), float(nets[k].blob("m").ravel()[0])
        sv, mv = views[k]
        record[0:1].copy_(sv)       # float -> double on the device
        record[1:2].copy_(mv)
        comm.allgather_records(record, gathered, torch.cuda.current_stream().cuda_stream)
        landing.copy_(gathered, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        g = landing.numpy()
        return float(np.sum(g[0::2])), float(np.max(g[1::2]))   # rank order

    res = None
    with cf.ThreadPoolExecutor(max_workers=2) as pool:
        total = warmup + steps
        pending = {}
        for i in range(min(2, total)):
            pending[i] = pool.submit(forward, i % 2)
        t0 = None
        for i in range(total):
            if i == warmup:
                t0 = time.perf_counter()
            pending.pop(i).result()
            res = results(i % 2)
            if i + 2 < total:
                pending[i + 2] = pool.submit(forward, i % 2)
        dt = time.perf_counter() - t0
    if comm is not None:
        tmax = torch.tensor([dt], dtype=torch.float64, device=device)
        comm.allreduce_partials(tmax, RED_MAX, torch.cuda.current_stream().cuda_stream)
        dt = float(tmax.item())
    h2d = a_host.numel() * 4 + b_host.numel() * 4
    d2h = 8 if world == 1 else 16 * world
    return dt / steps, h2d, d2h, res


def run_b200_arm(args):
    global A_SHAPE, O_SHAPE
    if args.batch != A_SHAPE[0]:
        A_SHAPE, O_SHAPE = (args.batch,) + A_SHAPE[1:], (args.batch,) + O_SHAPE[1:]
    import torch
    from shadow_b200 import capi, sharded
    from shadow_b200 import functional as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist, comm = None, None
    json_out = sys.stdout
    if world > 1:
        import torch.distributed as dist
        # NCCL writes its version banner to the process's stdout whatever NCCL_DEBUG_FILE says: move
        # file descriptor 1 to stderr for the run and keep the real stdout for the one JSON line
        sys.stdout.flush()
        json_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL's communicator set-up lines (rank count, transport) are wanted in the log: INFO level for the INIT
        # subsystem.  NCCL writes them to the process's stdout, which points at stderr for this run (above), so
        # stdout proper stays the one JSON line.
        if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
            os.environ["NCCL_DEBUG"] = "INFO"
        os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
        os.environ.pop("NCCL_DEBUG_FILE", None)
        # a rank that stalls in a collective must not keep 8 GPUs busy: the whole run takes well
        # under a minute, so after 3 minutes the process ends itself
        safety = threading.Timer(180.0, os._exit, args=(3,))
        safety.daemon = True
        safety.start()
        torch.cuda.set_device(local_rank)
        # torch.distributed carries the rendezvous (the 128-byte identifier, barriers); the data path's
        # one exchange goes through the C entry points of libsb200_nccl.so on its own communicator
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))
        from shadow_b200.comm import Communicator
        comm = Communicator.from_process_group()
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node %d" % args.gpus
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    capi.lib()   # fail loudly now if the CUDA library is missing

    # ---- synthetic inputs: the rank's dim-0 slab of A (pinned on the host, then resident in HBM)
    a_np, b_np = make_inputs(A_SHAPE, B_SHAPE)
    lo, hi = sharded.shard_bounds(A_SHAPE[0], rank, world)
    a_host = torch.from_numpy(np.ascontiguousarray(a_np[lo:hi])).pin_memory()
    b_host = torch.from_numpy(b_np).pin_memory()
    del a_np
    n_local = hi - lo
    A = a_host.to(device, non_blocking=True)
    B = b_host.to(device, non_blocking=True)
    O = torch.empty((n_local,) + O_SHAPE[1:], dtype=torch.float32, device=device)
    torch.cuda.synchronize()

    # Steps are captured `chunk` at a time (the largest divisor of --steps up to 10), each with its
    # own record slot, so that the exchange of step i can run beside the Mul of step i+1.
    chunk = 1
    if world > 1 and not args.no_graph:
        chunk = max(c for c in range(1, 11) if args.steps % c == 0)
    total = numel(O_SHAPE)
    # the package's sharded reduction: both reductions behind ONE all-gather of 16 bytes per rank,
    # folded in rank order on every rank (sharded.ReduceMany over the C entry points)
    many = sharded.ReduceMany([RED_SUM, RED_MAX], (n_local,) + O_SHAPE[1:], [], O_SHAPE[0], device, comm=comm, slots=chunk)
    # the 16-byte exchange must not queue behind a full-GPU kernel: highest priority
    side = torch.cuda.Stream(device=device, priority=-1) if world > 1 else None

    def step(slot=0, overlap=False):
        """One pass of the chain.  With `overlap` the exchange and the fold go to the side stream that
        the caller joins later (many.join()), so the next step's Mul does not wait for them."""
        F.binary(A, B, MUL, out=O)
        many(O, slot=slot, side_stream=side if overlap else None)

    def step_with_events(evs):
        """The three kernels of a rank's step launched directly with events between them (the
        exchange is left out: per-operator durations)."""
        evs[0].record()
        F.binary(A, B, MUL, out=O)
        evs[1].record()
        if world == 1:
            F.reduce(O, RED_SUM, [], out=many.results[0][0])
            evs[2].record()
            F.reduce(O, RED_MAX, [], out=many.results[0][1])
        else:
            F.reduce_partial(O, RED_SUM, [], out=many.records[0][0:1])
            evs[2].record()
            F.reduce_partial(O, RED_MAX, [], out=many.records[0][1:2])
        evs[3].record()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    # ---- the step as a CUDA graph: the launches (and the collective) are captured once and the
    # timed region replays them, so the host cost per step is one graph launch
    graph = None
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        launches_before = capi.launch_count()
        with torch.cuda.graph(graph):
            for c in range(chunk):
                step(slot=c, overlap=chunk > 1)
            if chunk > 1:
                many.join()   # every exchange of the chunk has finished
        launches_per_step = (capi.launch_count() - launches_before) // chunk
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()

    def run_chunk():
        """`chunk` steps (one graph replay), or one directly launched step."""
        if graph is not None:
            graph.replay()
        else:
            step()

    # the clock sampler is a child process: it is started (and has reported once) BEFORE the barrier, so that
    # nothing but the timed launches lies between the barrier and the timed region
    clocks = ClockSampler(local_rank, ready_wait_s=0.0 if args.no_clocks else 15.0)
    clocks.__enter__()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    launches_before = capi.launch_count()

    def timed_block():
        """EXACTLY args.steps steps between two events; max over ranks of the device time."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(args.steps // chunk):
            run_chunk()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        if dist is not None:
            tmax = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            ms = float(tmax.item())
        return ms

    try:
        ms_total = timed_block()          # the reported number: the first block of exactly --steps steps
        # The same block again, several times: a timed region of a few milliseconds yields no clock
        # samples and says nothing about run-to-run spread.  The count derives from the max-over-ranks
        # time, so every rank runs the same number of blocks (each step holds a collective).
        repeats = [ms_total]
        if not args.no_clocks:
            n_more = int(min(200, max(4, 300.0 / max(ms_total, 1e-3))))
            for _ in range(n_more):
                repeats.append(timed_block())
    finally:
        clocks.__exit__(None, None, None)
    extra = (len(repeats) - 1) * args.steps
    launches = (launches_per_step * args.steps) if graph is not None else (capi.launch_count() - launches_before) // len(repeats)
    if dist is not None:
        dist.barrier()
    last = (chunk - 1) if graph is not None else 0
    r_sum, r_max = many.results[last]
    s, m = r_sum.clone(), r_max.clone()
    # ---- self-check of the sharded result: every rank's double partials of the last step, brought to
    # the host once and folded there in rank order, must give the bits the device path produced
    results_check = None
    if world > 1:
        mine = many.records[last].clone()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        host = np.stack([p.cpu().numpy() for p in parts])            # [rank, (sum, max)]
        acc = 0.0
        for r in range(world):
            acc += float(host[r, 0])
        want_sum, want_max = float(np.float32(acc)), float(np.float32(host[:, 1].max()))
        results_check = {"sum_from_rank_partials": want_sum, "max_from_rank_partials": want_max,
                         "matches": bool(want_sum == float(s.item()) and want_max == float(m.item()))}
        if rank == 0:
            # and against the whole (unsharded) tensor on the host: float products as the operator forms them,
            # summed in double, slice by slice (a few seconds of numpy on rank 0, outside every timed region)
            a_full, b_full = make_inputs(A_SHAPE, B_SHAPE)
            host_sum, host_max = 0.0, -np.inf
            for n in range(A_SHAPE[0]):
                o = a_full[n] * b_full[0]            # [1,2048,2048] x [16,1,2048] -> [16,2048,2048] float32
                host_sum += float(np.sum(o, dtype=np.float64))
                host_max = max(host_max, float(o.max()))
            tol = 1e-5 * np.log2(numel(O_SHAPE))
            results_check.update({"host_double_sum": host_sum, "host_max": host_max,
                                  "agrees_with_unsharded_host": bool(abs(float(s.item()) - host_sum) <= tol * abs(host_sum)
                                                                     and float(m.item()) == host_max)})
            del a_full, b_full, o

    # ---- per-operator durations: the same steps launched directly with CUDA events between the
    # operators (events cannot be read inside a graph replay)
    n_inst = max(3, min(args.steps, 20))
    op_events = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_inst)]
    for k in range(n_inst):
        step_with_events(op_events[k])
    torch.cuda.synchronize()
    ms_step = ms_total / args.steps
    bytes_job = step_bytes(A_SHAPE, B_SHAPE, O_SHAPE)          # whole job, all ranks
    bytes_rank = step_bytes((n_local,) + A_SHAPE[1:], B_SHAPE, (n_local,) + O_SHAPE[1:])
    value = sum(bytes_job.values()) / ms_step / 1e6
    op_ms = {
        "binary_broadcast_mul": statistics.mean(e[0].elapsed_time(e[1]) for e in op_events),
        "reduce_sum_all": statistics.mean(e[1].elapsed_time(e[2]) for e in op_events),
        "reduce_max_all": statistics.mean(e[2].elapsed_time(e[3]) for e in op_events),
    }
    peak, peak_kind = measured_peak()
    mul_gbs = bytes_rank["binary_broadcast_mul"] / op_ms["binary_broadcast_mul"] / 1e6
    roofline = {"bound": "hbm", "kernel": "bcast_reuse_kernel (broadcast Mul, per rank)", "achieved": round(mul_gbs, 1),
                "peak": peak, "peak_source": "MEASURED_PEAKS.json hbm_gbs" if peak_kind == "measured" else "fallback",
                "unit": "GB/s", "frac": round(mul_gbs / peak, 4), "frac_of_8tbs": round(mul_gbs / NOMINAL_PEAK_GBS, 4),
                "traffic": ncu_traffic()}
    per_step_ops = {k: {"ms": round(v, 4), "gb_per_s_per_gpu": round(bytes_rank[k] / v / 1e6, 1)} for k, v in op_ms.items()}
    result_sum, result_max = float(s.item()), float(m.item())

    # ---- end to end through the Network API with host buffers
    if args.no_e2e:
        e2e_s, h2d, d2h, e2e_res = float("nan"), 0, 0, (None, None)
    else:
        e2e_s, h2d, d2h, e2e_res = run_e2e(n_local, local_rank, a_host, b_host, max(4, min(args.steps, 20)), 4, comm, torch)
    e2e_value = sum(bytes_job.values()) / e2e_s / 1e9

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C5 chain: broadcast Mul A[8,1,2048,2048]xB[1,16,1,2048] -> [8,16,2048,2048] (2 GiB), "
                               "ReduceSum all axes, ReduceMax all axes; dim 0 split over the ranks",
                   "l2": "inputs larger than L2 (each step streams >= 256 MiB per GPU; no flush interposed)",
                   "bytes_per_step": sum(bytes_job.values()),
                   "collective": ("one NCCL all-gather of 16 B per rank per step (sum and max partials together) through the C entry "
                                  "sb200_sharded_reduce_finish (sharded.ReduceMany)"
                                  + (", on a side stream beside the next step's Mul" if chunk > 1 else "")) if world > 1 else "none",
                   "launch": ("cuda graph replay, %d steps per graph" % chunk) if graph is not None else "direct launches"},
        "frac_of_8tbs_per_gpu": round(value / world / NOMINAL_PEAK_GBS, 4),
        "roofline": roofline, "per_step_ops": per_step_ops,
        "e2e": None if args.no_e2e else {"value": round(e2e_value, 3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_s * 1e3, 3),
                "api": "Shadow::Network::Forward + GetBlobDataByName (C++ host library); two Networks on two host threads "
                       "take the steps alternately" + ("; ranks combine through sb200_allgather_records" if world > 1 else "")},
        "gpu_launches": launches,
        "clocks": dict(clocks.summary(), window="timed region + %d identical steps (the repeats)" % extra),
        "repeats": {"blocks": len(repeats), "steps_per_block": args.steps,
                    "ms_per_step_min": round(min(repeats) / args.steps, 4),
                    "ms_per_step_median": round(statistics.median(repeats) / args.steps, 4),
                    "ms_per_step_max": round(max(repeats) / args.steps, 4),
                    "note": "value and ms_per_step are the FIRST block; the others repeat it under the clock sampler"},
        "results": {"sum": result_sum, "max": result_max, "e2e_sum": e2e_res[0], "e2e_max": e2e_res[1]},
    }
    if results_check is not None:
        line["results_check"] = results_check
    if rank == 0 and world == 1:
        if not args.no_sweep:
            line["per_op_256mb"] = per_op_sweep(torch, F, device, peak)
        if not args.no_cpu:
            gbs, ms, kind, _, a_sample, cpu_res = time_cpu(1, 3, 1, slices=1)
            # the same sample on the GPU, against the CPU result: parity of what was timed
            As = torch.from_numpy(a_sample).to(device)
            Os = F.binary(As, B, MUL)
            gs = float(F.reduce(Os, RED_SUM, [], False).item())
            gm = float(F.reduce(Os, RED_MAX, [], False).item())
            tol = 1e-5 * np.log2(numel(SAMPLE_O))
            line["cpu_baseline"] = {"value": round(gbs, 4), "unit": UNIT, "cores": 1, "kind": kind,
                                    "sample": SAMPLE_TEXT, "ms_per_sample_step": round(ms, 2),
                                    "sample_parity": bool(abs(gs - cpu_res[0]) <= tol * abs(cpu_res[0]) and gm == cpu_res[1])}
    if rank == 0:
        print(json.dumps(line), file=json_out, flush=True)
    # ---- teardown.  Everything has been reported; a collective captured in a CUDA graph must be
    # released before the communicator goes away, and a teardown that stalls must not keep the job
    # (and the GPUs) alive: after 20 s the process exits on its own.
    if dist is not None:
        watchdog = threading.Timer(20.0, os._exit, args=(0,))
        watchdog.daemon = True
        watchdog.start()
        if graph is not None:
            graph.reset()
        graph = None
        torch.cuda.synchronize()
        dist.barrier()
        if comm is not None:
            comm.close()
        dist.destroy_process_group()
        watchdog.cancel()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-operator >=256 MB sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch every step directly instead of replaying a CUDA graph")
    ap.add_argument("--no-clocks", action="store_true", help="do not prolong the loop for clock sampling")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffers) leg")
    ap.add_argument("--batch", type=int, default=A_SHAPE[0],
                    help="dim 0 of A (default 8 = the baseline configuration; smaller only for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_b200_arm(args)


if __name__ == "__main__":
    sys.exit(main())

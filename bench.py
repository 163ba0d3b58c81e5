#!/usr/bin/env python
"""Benchmark of the Ferrox training hot path on B200: CNN train-step images/sec.

Workload: the deeper CNN of the baseline configuration — global batch 1024 x 3 x 32 x 32 (values
N(0,1), seeded), labels uniform in [0,10), four conv 3x3 pad 1 layers 3->64->128->256->256 with
bias + ReLU (stride 2 on layers 2-4), flatten (4096), linear 4096->10, softmax cross-entropy,
Adam(lr=1e-3).  One step = forward + backward + gradient all-reduce (N > 1) + optimizer step.
The global batch is fixed and sharded evenly over the ranks (strong scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case NAME [--dtype f32|f64] [--launches N]     # one kernel case (timing / profiling)
    python bench.py --phases [--gpus N]                              # per-phase timeline of the train step

With N > 1 it is launched as `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N`.
Rank 0 prints one JSON line.  At N = 1 the line also carries `configs`: the single-layer convolution sweep
(forward, input gradient, filter gradient; f32 and f64), the MLP step and the HBM microbenchmark shapes of the
other baseline configurations, each with its fraction of the measured roof.  `--impl reference` times the
reference's CPU path (the single-threaded restatement under oracle/, since the Rust reference cannot be
built here) on a bounded sample.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GLOBAL_BATCH = 1024
SEED = 20261125
METRIC = "CNN train-step images/sec"
UNIT = "images/s"
CPU_SAMPLE_IMAGES = 32
# conv/linear contraction FLOPs of one train step, per image (2*M*N*K of each implicit GEMM of the
# deep CNN: conv 3->64 on 32x32, 64->128 on 16x16, 128->256 on 8x8, 256->256 on 4x4 outputs, linear
# 4096->10; forward + dX + dW, no dX for the first layer).
FWD_FLOP_PER_IMAGE = 3538944 + 37748736 + 37748736 + 18874368 + 81920
STEP_FLOP_PER_IMAGE = 3 * FWD_FLOP_PER_IMAGE - 3538944
# fallbacks used only when the measured-peaks file is absent (an earlier measurement on this kind of GPU)
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def synthetic_batch(rng, n, dtype=np.float32):
    x = rng.standard_normal((n, 3, 32, 32)).astype(dtype)
    labels = rng.integers(0, 10, n)
    return x, np.eye(10, dtype=dtype)[labels]


def workload_config(world, graph=False):
    """The `config` object of the JSON line (the same for both arms)."""
    return {"workload": "deep_cnn_train_step_global_batch_1024", "global_batch": GLOBAL_BATCH,
            "per_gpu_batch": GLOBAL_BATCH // world, "optimizer": "adam", "math": "3xTF32 on tcgen05, f32 accumulate",
            "parallelism": f"dp{world}", "l2": "256 MiB buffer written, then a second 256 MiB read, between timed steps (not timed)",
            "allreduce": "NCCL sum, 2 buckets (last layers holding half of the parameters first), overlapped with backward"
                         if world > 1 else "none"}


def measured_peaks():
    """HBM GB/s and dense bf16 TFLOP/s measured on this pool's GPUs (a file written next to this script by
    the harness that runs the benchmark), else the fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "of measured"}
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "source": "of fallback"}


# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # the busiest half of the samples is "under load"
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": float(np.median(load)) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU baselines
def cpu_reference_step_rate(sample_images, steps, warmup):
    """(images/s, seconds per step) of the reference CPU path (single-threaded restatement) on
    `sample_images` images per step."""
    from oracle import cpu_oracle as orc
    from ferrox_b200.train import deep_cnn_layers, kaiming_uniform_params
    layers, in_shape = deep_cnn_layers()
    acts = {None: 0, "relu": 1}
    ol = [dict(kind=L["kind"], stride=L.get("stride", 1), pad=L.get("pad", 0), act=acts[L.get("act")]) for L in layers]
    rng = np.random.default_rng(SEED)
    params = kaiming_uniform_params(layers, in_shape, rng, np.float32)
    m = [(np.zeros_like(w), np.zeros_like(b)) for w, b in params]
    v = [(np.zeros_like(w), np.zeros_like(b)) for w, b in params]
    x, t = synthetic_batch(rng, sample_images)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        _, grads = orc.net_forward_backward(ol, params, x, t)
        for i, ((w, b), (gw, gb)) in enumerate(zip(params, grads)):
            orc.adam_step(w.reshape(-1), gw.reshape(-1), m[i][0].reshape(-1), v[i][0].reshape(-1), it + 1, lr=1e-3)
            orc.adam_step(b.reshape(-1), gb.reshape(-1), m[i][1].reshape(-1), v[i][1].reshape(-1), it + 1, lr=1e-3)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    return sample_images / float(np.mean(times)), float(np.mean(times))


def torch_cpu_step_rate(sample_images=256, steps=2, warmup=1):
    """images/s of the same train step written with torch's CPU autograd on all host cores.  This is NOT the
    reference (Ferrox's CPU path is single-threaded ndarray code); it is a stronger CPU baseline for context."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(SEED)
    chans = [3, 64, 128, 256, 256]
    ws = [torch.tensor((rng.uniform(-1, 1, (chans[i + 1], chans[i], 3, 3)) * np.sqrt(6.0 / (chans[i] * 9))).astype(np.float32),
                       requires_grad=True) for i in range(4)]
    bs = [torch.zeros(chans[i + 1], requires_grad=True) for i in range(4)]
    wf = torch.tensor((rng.uniform(-1, 1, (10, 4096)) * np.sqrt(6.0 / 4096)).astype(np.float32), requires_grad=True)
    bf = torch.zeros(10, requires_grad=True)
    params = ws + bs + [wf, bf]
    opt = torch.optim.Adam(params, lr=1e-3)
    xs, ts = synthetic_batch(rng, sample_images)
    x, lab = torch.from_numpy(xs), torch.from_numpy(ts.argmax(1))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        h = x
        for i, s in enumerate((1, 2, 2, 2)):
            h = F.relu(F.conv2d(h, ws[i], bs[i], stride=s, padding=1))
        loss = F.cross_entropy(F.linear(h.flatten(1), wf, bf), lab)
        opt.zero_grad()
        loss.backward()
        opt.step()
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return sample_images / float(np.mean(times)), torch.get_num_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    rate, sec = cpu_reference_step_rate(CPU_SAMPLE_IMAGES, args.steps, args.warmup)
    sample = (f"each step = forward + backward + Adam on {CPU_SAMPLE_IMAGES} of the {GLOBAL_BATCH} images of the global batch; "
              "single-threaded C++ restatement of the reference's ndarray path (the reference's CPU path is single-threaded; "
              "the Rust toolchain is absent, so the reference itself cannot be built); its GEMM is a blocked triple loop, "
              "slower than the SIMD micro-kernel of the matrixmultiply crate the reference calls")
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(max(1, args.gpus)),
        "sample_images": CPU_SAMPLE_IMAGES,
        "ms_per_global_batch_extrapolated": sec * 1e3 * GLOBAL_BATCH / CPU_SAMPLE_IMAGES,
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ peaks and kernel cases
def measure_gemm_peak(dtype_name):
    """Dense GEMM throughput of the vendor library on this GPU, TFLOP/s: TF32 (the roofline denominator of the
    f32 contractions is a third of it, 3xTF32 issues three MMAs per product) or f64."""
    import torch
    f64 = dtype_name == "f64"
    n = 4096 if f64 else 8192
    dt = torch.float64 if f64 else torch.float32
    a = torch.randn(n, n, device="cuda", dtype=dt)
    b = torch.randn(n, n, device="cuda", dtype=dt)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        best = 0.0
        for i in range(8):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                best = max(best, 2.0 * n ** 3 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    return best


CONV_LAYERS = {  # name -> N, C, H, W, K, stride (3x3 filters, pad 1)
    "c3a": (128, 64, 56, 56, 64, 1),      # single-layer sweep, first point
    "c3b": (64, 256, 14, 14, 512, 2),     # single-layer sweep, second point
    "conv1": (1024, 3, 32, 32, 64, 1),    # layers of the deep CNN at batch 1024
    "conv2": (1024, 64, 32, 32, 128, 2),
    "conv3": (1024, 128, 16, 16, 256, 2),
    "conv4": (1024, 256, 8, 8, 256, 2),
}
CASE_ALIASES = {"conv_fwd": "conv2_fwd", "conv_dgrad": "conv2_dgrad", "conv_wgrad": "conv2_wgrad", "conv3a": "c3a_fwd"}


def list_cases():
    names = [f"{k}_{p}" for k in CONV_LAYERS for p in ("fwd", "dgrad", "wgrad")]
    names += ["gemm", "matmul_no_workspace", "mlp_step", "act_bwd_relu", "act_bwd_sigmoid", "act_bwd_tanh", "act_bwd_small", "colsum", "colsum_small",
              "chansum", "transpose", "bn_fwd", "bn_bwd", "gap_fwd", "softmax_ce", "adam", "linear_head"]
    return names + list(CASE_ALIASES)


def make_case(name, ops, dev, dtype_name):
    """Returns (fn, work, unit): one call of `fn` does `work` units (1e12 FLOP or 1e9 bytes, algorithmic)."""
    import torch
    name = CASE_ALIASES.get(name, name)
    dt = torch.float32 if dtype_name == "f32" else torch.float64
    es = 4 if dtype_name == "f32" else 8
    g = torch.Generator(device=dev).manual_seed(SEED)

    def randn(*shape):
        return torch.randn(*shape, device=dev, dtype=dt, generator=g)

    head, _, part = name.rpartition("_")
    if head in CONV_LAYERS and part in ("fwd", "dgrad", "wgrad"):
        N, C, H, W, K, s = CONV_LAYERS[head]
        x = randn(N, C, H, W)
        w = randn(K, C, 3, 3) * float(np.sqrt(2.0 / (C * 9)))
        b = randn(K) * 0.1
        y = ops.conv2d_forward(x, w, (s, s), (1, 1), b, "relu")
        dy = randn(*y.shape)
        work = 2.0 * y.numel() * C * 9 / 1e12
        fn = {"fwd": lambda: ops.conv2d_forward(x, w, (s, s), (1, 1), b, "relu"),
              "dgrad": lambda: ops.deconv2d(dy, w, x.shape, (s, s), (1, 1), y, "relu"),
              "wgrad": lambda: ops.cross_correlation2d(x, dy, w.shape, (s, s), (1, 1), y, "relu", want_bias_grad=True)}[part]
        return fn, work, "TFLOP/s"
    if name == "gemm":
        n = 4096 if dtype_name == "f32" else 2048
        A, B = randn(n, n), randn(n, n)
        return (lambda: ops.linear_forward(A, B)), 2.0 * n ** 3 / 1e12, "TFLOP/s"
    if name == "matmul_no_workspace":
        # fxb_matmul has no workspace argument: the first-generation engine (thread-fed operands) at the same size
        n = 4096 if dtype_name == "f32" else 2048
        A, B, C = randn(n, n), randn(n, n), randn(n, n)
        fnc = ops._fn("matmul", A)
        from ctypes import c_void_p
        pa, pb, pc = c_void_p(A.data_ptr()), c_void_p(B.data_ptr()), c_void_p(C.data_ptr())

        def call():
            ops._check(fnc(ops.h, pa, pb, pc, n, n, n, ops._stream()))
        call.keepalive = (A, B, C)
        return call, 2.0 * n ** 3 / 1e12, "TFLOP/s"
    if name == "mlp_step":
        from ferrox_b200.train import SequentialNet, kaiming_uniform_params, mlp_layers
        layers, in_shape = mlp_layers()
        net = SequentialNet(ops, layers, 256, in_shape, dt)
        net.set_params(kaiming_uniform_params(layers, in_shape, np.random.default_rng(SEED), np.float32 if es == 4 else np.float64))
        x = randn(256, 784)
        t = torch.eye(10, device=dev, dtype=dt)[torch.randint(0, 10, (256,), device=dev, generator=g)]

        def step():
            net.forward(x)
            net.loss(t)
            net.backward_range(x, net.n_param_layers - 1, 0)
        step.keepalive = net
        return step, 1027080192 / 1e12, "TFLOP/s"
    if name.startswith("act_bwd"):
        kind = name.split("_")[2]
        n = 1 << (26 if kind == "small" else 28)
        act = "relu" if kind == "small" else kind
        aux, dy = randn(n), randn(n)
        if act != "relu":
            aux = getattr(ops, act)(aux)
        return (lambda: ops.act_backward(dy, aux, act)), 3.0 * n * es / 1e9, "GB/s"
    if name in ("colsum", "colsum_small"):
        x = randn(65536 if name == "colsum" else 16384, 4096)
        return (lambda: ops.sum_axes(x, [0])), x.numel() * es / 1e9, "GB/s"
    if name == "chansum":
        x = randn(256, 64, 56, 56)
        return (lambda: ops.sum_axes(x, [0, 2, 3])), x.numel() * es / 1e9, "GB/s"
    if name == "transpose":
        x = randn(8192, 8192)
        return (lambda: ops.transpose(x)), 2.0 * x.numel() * es / 1e9, "GB/s"
    if name in ("bn_fwd", "bn_bwd"):
        x = randn(256, 64, 56, 56)
        ga, be = randn(64), randn(64)
        y, mean, var = ops.batch_norm_forward(x, ga, be, 1e-3, 0.1, None, None, True, "relu")
        dy = randn(*x.shape)
        if name == "bn_fwd":  # two statistics passes and the normalising pass read x, one write
            return (lambda: ops.batch_norm_forward(x, ga, be, 1e-3, 0.1, None, None, True, "relu")), 4.0 * x.numel() * es / 1e9, "GB/s"
        # the reduction pass reads x, dy, y; the apply pass reads them again and writes dx
        return (lambda: ops.batch_norm_backward(x, dy, ga, mean, var, 1e-3, y, "relu")), 7.0 * x.numel() * es / 1e9, "GB/s"
    if name == "gap_fwd":
        x = randn(1024, 256, 28, 28)
        return (lambda: ops.global_avg_pool_forward(x)), x.numel() * es / 1e9, "GB/s"
    if name == "softmax_ce":
        z = randn(1 << 20, 10)
        t = torch.eye(10, device=dev, dtype=dt)[torch.randint(0, 10, (1 << 20,), device=dev, generator=g)]
        return (lambda: ops.softmax_cross_entropy(z, t)), 3.0 * z.numel() * es / 1e9, "GB/s"
    if name == "adam":
        n = 1 << 26
        p, gr, m, v = randn(n), randn(n), torch.zeros(n, device=dev, dtype=dt), torch.zeros(n, device=dev, dtype=dt)
        return (lambda: ops.adam_step_(p, gr, m, v, 1)), 7.0 * n * es / 1e9, "GB/s"
    if name == "linear_head":  # the classifier of the deep CNN at batch 1024: forward + backward
        X, Wt, b = randn(1024, 4096), randn(10, 4096) * 0.02, randn(10)
        dy = randn(1024, 10)

        def fn():
            ops.linear_forward(X, Wt, b)
            ops.linear_backward(X, Wt, dy)
        return fn, 3 * 2.0 * 1024 * 4096 * 10 / 1e12, "TFLOP/s"
    raise SystemExit(f"unknown case {name}; cases: {' '.join(list_cases())}")


class L2Flush:
    """Evicts the 126 MB L2 between timed iterations (not timed): writes a 256 MiB buffer, then reads a second one,
    so that the timed kernels start from a cold L2 that holds none of the flush's own dirty lines (their write-back
    would otherwise fall into the timed region)."""

    def __init__(self, dev):
        import torch
        self.w = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.r = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
        self.sink = None

    def __call__(self):
        self.w.zero_()
        self.sink = self.r.sum()


def time_case(fn, reps, flush=None):
    """Median CUDA-event time (ms) of `reps` calls, the L2 flushed before each (not timed)."""
    import torch
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush is not None:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts))


def run_case(args):
    import torch
    from ferrox_b200 import build
    build.build()
    from ferrox_b200.cuda_ops import CudaOps
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ops = CudaOps(0)
    if args.accumulate_stages:
        ops.set_accumulate_stages(args.accumulate_stages)
    if args.single_pass:
        ops.set_math_mode(1)
    fn, work, unit = make_case(args.case, ops, dev, args.dtype)
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status()
    ms = e0.elapsed_time(e1) / args.launches
    print(json.dumps({"case": args.case, "dtype": args.dtype, "launches": args.launches, "ms_per_call": ms,
                      "rate": work / (ms * 1e-3), "unit": unit}), flush=True)


def measure_configs(ops, dev, flush, peaks, tf32_peak, f64_peak):
    """The other baseline configurations on one GPU: per case ms (median of 5, L2 flushed), achieved rate
    and fraction of the roof (3xTF32 = measured TF32 GEMM / 3, f64 = measured f64 GEMM, streaming = measured HBM)."""
    import torch
    f32_roof = peaks["bf16_tflops"] / 2.0 / 3.0
    out = {"roofs": {"f32_3xtf32_tflops": f32_roof, "f64_tflops": f64_peak, "hbm_gbs": peaks["hbm_gbs"],
                     "tf32_gemm_in_run_tflops": tf32_peak,
                     "note": "f32 roof = dense bf16 GEMM " + peaks["source"] + " / 2 / 3 (3xTF32); f64 roof = torch.matmul f64 4096^3 "
                             "measured in this run (the peaks file has no f64 entry); HBM " + peaks["source"]}}
    plan = [(f"{k}_{p}", dts) for k in ("c3a", "c3b") for p in ("fwd", "dgrad", "wgrad") for dts in (("f32", "f64"),)]
    plan += [("gemm", ("f32", "f64")), ("mlp_step", ("f32",)), ("colsum", ("f32", "f64")), ("chansum", ("f32", "f64")), ("act_bwd_relu", ("f32", "f64")),
             ("act_bwd_sigmoid", ("f32", "f64")), ("act_bwd_tanh", ("f32", "f64"))]
    for name, dts in plan:
        for d in dts:
            fn, work, unit = make_case(name, ops, dev, d)
            ms = time_case(fn, 5, flush)
            rate = work / (ms * 1e-3)
            roof = (f32_roof if d == "f32" else f64_peak) if unit == "TFLOP/s" else peaks["hbm_gbs"]
            out[f"{name}_{d}"] = {"ms": ms, "rate": rate, "unit": unit, "frac": rate / roof if roof else None}
            del fn
            torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------ the train-step benchmark
def setup_training(rank, world, local_rank, use_graph=False, batch_override=None, bucket_splits=None):
    import torch
    import torch.distributed as dist
    from ferrox_b200 import build
    if rank == 0:
        build.build()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    from ferrox_b200.cuda_ops import CudaOps
    from ferrox_b200.train import SequentialNet, Trainer, deep_cnn_layers, kaiming_uniform_params
    assert GLOBAL_BATCH % world == 0
    local_b = batch_override or GLOBAL_BATCH // world
    ops = CudaOps(local_rank)
    layers, in_shape = deep_cnn_layers()
    rng = np.random.default_rng(SEED)
    params = kaiming_uniform_params(layers, in_shape, rng, np.float32)
    xg, tg = synthetic_batch(rng, GLOBAL_BATCH)
    net = SequentialNet(ops, layers, local_b, in_shape, torch.float32)
    net.set_params(params)
    tr = Trainer(net, optimizer="adam", lr=1e-3, world_size=world, use_graph=use_graph, bucket_splits=bucket_splits)
    first = 0 if batch_override else rank * local_b
    xs = np.ascontiguousarray(xg[first:first + local_b])
    ts = np.ascontiguousarray(tg[first:first + local_b])
    return dev, ops, net, tr, xs, ts, local_b


def run_phases(args, rank, world, local_rank):
    """Per-phase timeline of the train step on this rank: CUDA-event time of every phase (forward, loss, each
    layer's backward, each all-reduce wait, optimizer) and the host time spent issuing it, averaged over the steps."""
    import torch
    import torch.distributed as dist
    dev, ops, net, tr, xs, ts, local_b = setup_training(rank, world, local_rank, batch_override=args.batch, bucket_splits=args.bucket_splits)
    x_dev, t_dev = torch.from_numpy(xs).to(dev), torch.from_numpy(ts).to(dev)
    for _ in range(20):
        tr.step(x_dev, t_dev)
    torch.cuda.synchronize()
    acc = {}
    steps = max(args.steps, 5)
    for _ in range(steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        marks = tr.step_with_marks(x_dev, t_dev)
        torch.cuda.synchronize()
        for (name, e0, h0), (_, e1, h1) in zip(marks[:-1], marks[1:]):
            a = acc.setdefault(name, [0.0, 0.0])
            a[0] += e0.elapsed_time(e1)
            a[1] += (h1 - h0) * 1e3
    ops.check_device_status()
    if rank == 0:
        phases = {k: {"gpu_ms": v[0] / steps, "host_ms": v[1] / steps} for k, v in acc.items()}
        print(json.dumps({"phases": phases, "n_gpus": world, "per_gpu_batch": local_b, "steps": steps,
                          "gpu_ms_total": sum(v["gpu_ms"] for v in phases.values()),
                          "host_ms_total": sum(v["host_ms"] for v in phases.values())}), flush=True)
    teardown(world, tr, net)


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    dev, ops, net, tr, xs, ts, local_b = setup_training(rank, world, local_rank, use_graph=args.graph, bucket_splits=args.bucket_splits)
    x_pin, t_pin = torch.from_numpy(xs).pin_memory(), torch.from_numpy(ts).pin_memory()
    x_dev, t_dev = x_pin.to(dev), t_pin.to(dev)
    x_stage, t_stage = torch.empty_like(x_dev), torch.empty_like(t_dev)
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    flush = L2Flush(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps):
        total = 0.0
        barrier()
        for _ in range(steps):
            flush()  # evict L2 between timed iterations (not timed)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step_fn()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        barrier()
        t = torch.tensor([total], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step_resident():
        tr.step(x_dev, t_dev)

    def step_e2e():
        xb, tb = tr.input_buffers() if args.graph else (None, None)
        xb, tb = (x_stage, t_stage) if xb is None else (xb, tb)  # graph mode: copy straight into the graph's inputs
        xb.copy_(x_pin, non_blocking=True)
        tb.copy_(t_pin, non_blocking=True)
        loss = tr.step(xb, tb)
        loss_host.copy_(loss, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    # The clock sampler (nvidia-smi, 50 ms period) runs from the warm-up on: the warm-up is the same load as
    # the timed steps, and at 8 GPUs the timed region alone (20 steps of about 1 ms) is shorter than one sample.
    # A fixed number of extra warm-up steps (the same on every rank: each step holds collectives) keeps the
    # GPU under load long enough for a handful of samples.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3) + 150):
        step_resident()
    torch.cuda.synchronize()
    ops.check_device_status()
    l0 = ops.launch_count()
    ms_total = timed(step_resident, args.steps)
    # kernels of this library per step: counted at the C ABI (eager) or while the graph was captured (replay)
    launches = tr.launches_per_step if (args.graph and tr.launches_per_step) else (ops.launch_count() - l0) // args.steps
    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    loss_value = tr.loss_value()
    ops.check_device_status()

    value = GLOBAL_BATCH * args.steps / (ms_total * 1e-3)
    e2e_value = GLOBAL_BATCH * args.steps / (ms_e2e * 1e-3)

    if rank == 0:
        peaks = measured_peaks()
        # Dominant kernel: umma_tma_conv_kernel, the tcgen05 implicit-GEMM convolution fed by the tensor-map
        # copy engine.  Its largest single launch in this step is the layer-2 forward (64->128, stride 2,
        # 16x16 output) on this rank's batch.  The operand pre-pass runs first (untimed), then the contraction
        # kernel alone is timed with CUDA events, L2 flushed before each launch.
        k_x = torch.randn(local_b, 64, 32, 32, device=dev)
        k_w = torch.randn(128, 64, 3, 3, device=dev) * 0.05
        k_b = torch.zeros(128, device=dev)
        flop = 2.0 * local_b * 16 * 16 * 128 * 64 * 9
        for _ in range(3):
            ops.conv2d_forward(k_x, k_w, (2, 2), (1, 1), k_b, "relu")
        ops.conv2d_forward_prepass(k_x, k_w, (2, 2), (1, 1))
        kernel_ms = time_case(lambda: ops.conv2d_forward_main(k_x.shape, k_w.shape, (2, 2), (1, 1), k_b, "relu"), 20, flush)
        ops.conv2d_forward_prepass(k_x, k_w, (2, 2), (1, 1))
        prepass_ms = time_case(lambda: ops.conv2d_forward_prepass(k_x, k_w, (2, 2), (1, 1)), 10, flush)
        call_ms = time_case(lambda: ops.conv2d_forward(k_x, k_w, (2, 2), (1, 1), k_b, "relu"), 10, flush)
        achieved = flop / (kernel_ms * 1e-3) / 1e12
        tf32_peak = measure_gemm_peak("f32")
        # Denominator: the measured dense bf16 GEMM rate of this pool's GPUs (file written by the harness), / 2 for
        # TF32 operands, / 3 because 3xTF32 issues three MMAs per product.  The vendor library's TF32 GEMM measured
        # in this run (a lower figure) is reported beside it.
        peak = peaks["bf16_tflops"] / 2.0 / 3.0
        traffic = None
        prof = os.path.join(ROOT, "profiles", "umma_tma_conv_kernel_traffic.json")
        if os.path.exists(prof):
            try:
                traffic = json.load(open(prof)).get("dram_bytes_per_launch_conv2_b%d" % local_b)
            except Exception:
                traffic = None
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": traffic, "kernel": "umma_tma_conv_kernel<128> (conv 64->128 s2 forward, this step's batch)",
                    "kernel_ms": kernel_ms, "prepass_ms": prepass_ms, "call_ms": call_ms,
                    "call_tflops_with_prepass": flop / (call_ms * 1e-3) / 1e12,
                    "peak_source": f"dense bf16 GEMM {peaks['bf16_tflops']:.1f} TFLOP/s ({peaks['source']}) / 2 for TF32 / 3 for 3xTF32",
                    "tf32_gemm_in_run_tflops": tf32_peak,
                    "frac_of_tf32_gemm_in_run": achieved / (tf32_peak / 3.0),
                    "step_contraction_tflops": STEP_FLOP_PER_IMAGE * value / 1e12,
                    "step_frac": STEP_FLOP_PER_IMAGE * value / 1e12 / peak}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(world, args.graph),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(x_pin.numel() * 4 + t_pin.numel() * 4) * world,
                    "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches), "launch_mode": "CUDA graph replay" if args.graph else "eager launches",
            "clocks": clocks, "roofline": roofline, "loss": loss_value,
        }
        if world == 1:
            rate, sec = cpu_reference_step_rate(CPU_SAMPLE_IMAGES, 3, 1)
            line["cpu_baseline"] = {
                "value": rate, "unit": UNIT, "cores": 1, "kind": "port", "host_cores": os.cpu_count(),
                "sample": f"{CPU_SAMPLE_IMAGES} images per step, 3 steps after 1 warm-up ({sec:.3f} s per step); single-threaded C++ "
                          "restatement of the reference's ndarray path (the reference is single-threaded)"}
            try:
                trate, threads = torch_cpu_step_rate()
                line["cpu_baseline"]["torch_cpu_all_cores"] = {
                    "value": trate, "unit": UNIT, "threads": threads,
                    "note": "not the reference: the same step with torch CPU autograd on all host cores, 256 images per step"}
            except Exception as exc:  # the stronger baseline is context only
                line["cpu_baseline"]["torch_cpu_all_cores"] = {"error": str(exc)[:200]}
            if not args.no_configs:
                f64_peak = measure_gemm_peak("f64")
                line["configs"] = measure_configs(ops, dev, flush, peaks, tf32_peak, f64_peak)
                ops.check_device_status()
        print(json.dumps(line), flush=True)
    teardown(world, tr, net)


def teardown(world, tr, net):
    """Releases the graph before the communicator; a teardown that does not finish in 30 s ends the process
    (the result line is out by then)."""
    import torch
    import torch.distributed as dist
    tr.close()
    torch.cuda.synchronize()
    net.close()
    if world > 1:
        def _down():
            dist.barrier()
            dist.destroy_process_group()
        t = threading.Thread(target=_down, daemon=True)
        t.start()
        t.join(30)
        sys.stdout.flush()
        sys.stderr.flush()
        if t.is_alive():
            os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="time one kernel case instead of the train step (see list_cases)")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--phases", action="store_true", help="print the per-phase timeline of the train step")
    ap.add_argument("--no-configs", action="store_true", help="skip the single-layer / microbenchmark configurations")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="launch every kernel eagerly instead of replaying the step from a CUDA graph (captured after three eager steps)")
    ap.add_argument("--single-pass", action="store_true", help="--case only: one TF32 MMA per product instead of 3xTF32 (timing only)")
    ap.add_argument("--accumulate-stages", type=int, default=None, choices=[1, 2, 4],
                    help="--case only: K stages accumulated in TMEM between drains (library default 4)")
    ap.add_argument("--bucket-splits", type=lambda v: [int(t) for t in v.split(",") if t], default=None,
                    help="parameter layers at which an all-reduce bucket starts, e.g. 3,1 (default: the trainer's two buckets)")
    ap.add_argument("--batch", type=int, default=None, help="--phases only: per-GPU batch (e.g. 128, the share of one of 8 GPUs)")
    args = ap.parse_args()
    # keep stdout to the one JSON line: NCCL writes its version banner (NCCL_DEBUG=VERSION/WARN) to stdout
    if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
        os.environ.pop("NCCL_DEBUG")
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.case:
        run_case(args)
        return
    if world == 1 and args.gpus > 1:
        # convenience: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__), "--gpus", str(args.gpus),
               "--steps", str(args.steps), "--warmup", str(args.warmup)] + (["--phases"] if args.phases else []) + \
              ([] if args.graph else ["--no-graph"])
        sys.exit(subprocess.call(cmd))
    if args.phases:
        run_phases(args, rank, world, local_rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

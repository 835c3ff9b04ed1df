#!/usr/bin/env python
"""Benchmark of the predictive-coding train step (metric: train_step samples/sec).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c2|c1|c4|c5] [--depth D] [--precision fp32|tf32|mixed]

One "step" is one full ``train_step`` (settle T times, learn, final energy) on one batch of
synthetic data.  At N=1 the workload is the configuration the headline metric is quoted on:
DKPPCN, width 512, 2048 hidden layers, batch 1024, T=2, tanh, SGD for W and Psi, inputs
N(0,1), one-hot 10-class targets (it fits one GPU: about 30 GB).  Printed on rank 0: ONE
JSON line with

* ``value``     samples/s with x,y already resident in HBM (``train_step_device``), timed with
                CUDA events on the library's own stream, max over ranks;
* ``e2e``       the same metric through the public host-buffer call ``net.train_step(x, y, T)``
                (pinned staging + H2D of x,y and the D2H energy read inside the timed region);
* ``roofline``  the dominant kernel (the grouped forward GEMM of one settling pass) timed on
                its own with CUDA events: both floors are stated (three tensor passes against the
                measured dense bf16 peak, algorithmic bytes against the measured copy bandwidth
                of MEASURED_PEAKS.json) and ``bound`` is the larger one; ``traffic`` is the DRAM
                traffic measured with ncu per layer times the layers of the launch; at N > 1 the
                same launch over each rank's own layers, the slowest rank's figure reported;
* ``cpu_baseline`` the reference's own CPU code (oracle/_ref; numpy restatement if that is
                absent) on a bounded sample of the workload — the same network cut to a few
                layers, scaled to the full depth by the layer ratio;
* clocks and throttle reasons sampled through NVML every 50 ms during the timed region.

``--impl reference`` times only the CPU leg and prints the same line shape with
``"impl": "reference"``: every one of its K steps is one train step of a BOUNDED SAMPLE of the
workload (the same network cut to fewer hidden layers, chosen so that the K+W steps end within
a couple of minutes); ``ms_per_step`` is the measured time of such a sample step and ``value``
is scaled to the full depth by the ratio of algorithmic FLOPs (``"extrapolated": true`` and
the sample depth are stated at the top level of the line).

Multi-GPU (launched by torchrun, one rank per GPU): the deep stack is layer-sharded, strong
scaling; the line then also carries ``batch_sharded_c4``, the wide FullPCN workload
batch-sharded over the same ranks.
"""
from __future__ import annotations

import argparse
import json
import os

# The compiled reference runs OpenMP regions AND OpenBLAS's own thread pool; with OpenMP's
# default active spinning the two pools fight for the cores of a small host (measured: 6x
# slower at 8 threads on 8 hardware threads).  Must be set before libgomp is loaded.
os.environ.setdefault("OMP_WAIT_POLICY", "PASSIVE")
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (kind, input, hidden width, hidden count, terminal, batch, T, act, x distribution)
    "c3": dict(kind="dkp", inp=512, width=512, hidden=2048, out=10, batch=1024, T=2, act="tanh",
               x="normal", desc="DKPPCN 512-(512x2048)-10 tanh B1024 T2 SGD/SGD"),
    "c2": dict(kind="dkp", inp=784, width=256, hidden=8, out=10, batch=256, T=2, act="tanh",
               x="uniform", desc="DKPPCN 784-(256x8)-10 tanh B256 T2 SGD/SGD"),
    "c1": dict(kind="simple", inp=784, width=128, hidden=2, out=10, batch=64, T=20, act="sigmoid",
               x="uniform", desc="SimplePCN 784-128-128-10 sigmoid B64 T20 SGD"),
    "c4": dict(kind="full", inp=3072, width=1024, hidden=4, out=10, batch=4096, T=20, act="gelu",
               x="normal", desc="FullPCN 3072-(1024x4)-10 gelu CE Adam B4096 T20"),
}
HYPER = dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0)
# C5: the reference has no pooling layer, so the 2x2 average pools of the named configuration
# are folded into stride-2 convolutions (3x3, pad 1); the dense 2048-10 head is a 4x4 convolution.
C5 = dict(input_shape=(3, 32, 32), batch=128, T=10, act="relu",
          convs=[(32, 3, 3, 2, 2, 1, 1), (64, 3, 3, 2, 2, 1, 1), (128, 3, 3, 2, 2, 1, 1),
                 (10, 4, 4, 1, 1, 0, 0)],
          desc="SimpleConvolutionalPCN 32x32x3 conv3x3/s2 32-64-128 + dense 2048-10 relu B128 T10 SGD")


def sizes_of(w, hidden=None):
    h = w["hidden"] if hidden is None else hidden
    return [w["inp"]] + [w["width"]] * h + [w["out"]]


def synth(w, sizes, seed=1234, wseed=99):
    """Seeded synthetic batch and explicitly set parameters (default init std of the
    reference layers; Psi ~ N(0, 1/fan_in) for the DKP configs)."""
    rng = np.random.default_rng(seed)
    B = w["batch"]
    x = (rng.random((B, sizes[0]), dtype=np.float32) if w["x"] == "uniform"
         else rng.normal(size=(B, sizes[0])).astype(np.float32))
    y = np.eye(sizes[-1], dtype=np.float32)[rng.integers(0, sizes[-1], B)]
    wr = np.random.default_rng(wseed)
    params = []
    for l in range(len(sizes) - 1):
        s, n = sizes[l], sizes[l + 1]
        p = {"W": wr.normal(0, np.sqrt(2.0 / (s + n)), (n, s)).astype(np.float32)}
        if w["kind"] != "simple":
            p["Psi"] = wr.normal(0, np.sqrt(1.0 / s), (s, sizes[-1])).astype(np.float32)
        params.append(p)
    return x, y, params


from deepity_b200.flops import algorithmic_flops  # noqa: E402


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled every 50 ms while the timed region runs.
    Reads through NVML in-process (nvidia_ml_py); one nvidia-smi process per sample is the
    fallback (slow, and eight of them at once on an 8-GPU host get in the ranks' way)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index=0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.index = index
        self.source = None
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                try:
                    idx = int(visible.split(",")[self.index])
                except ValueError:
                    pass
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)

    def _run_nvml(self):
        nv, h = self._nvml_handle()
        self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                "sw_power_cap": 0x4}
        self.source = "nvml"
        while not self._stop.is_set():
            self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
            mask = int(get_reasons(h))
            for nm, bit in bits.items():
                if mask & bit:
                    self.reasons.add(nm)
            self._stop.wait(0.05)

    def _run_smi(self):
        self.source = "nvidia-smi"
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip().split(",")
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
                for nm, v in zip(self.NAMES, out[2:]):
                    if v.strip().lower().startswith("active"):
                        self.reasons.add(nm)
            except Exception:
                pass
            self._stop.wait(0.2)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "source": self.source}


# ------------------------------------------------------------------------------ CPU leg
def host_cpu_info():
    """What bounds the CPU arm on this host: the affinity mask and the cgroup CPU quota."""
    info = {"affinity_cpus": len(os.sched_getaffinity(0)), "os_cpu_count": os.cpu_count(),
            "cgroup_cpu_quota": None, "omp_wait_policy": os.environ.get("OMP_WAIT_POLICY")}
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()[:2]
        if quota != "max":
            info["cgroup_cpu_quota"] = float(quota) / float(period)
    except Exception:
        pass
    return info


def _cpu_net(w, hidden):
    """The reference network (or its numpy restatement) cut to `hidden` hidden layers, with
    the benchmark's seeded parameters; returns (run one step, kind, x, y)."""
    from oracle import ref as oref
    sizes = sizes_of(w, hidden)
    x, y, params = synth(w, sizes)
    opts = {}
    if w["kind"] == "full":
        opts = dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM")
    if oref.available():
        kind = "reference"
        net = oref.RefNet(w["kind"], sizes, w["batch"], act=w["act"], options=opts, **HYPER)
    else:
        from oracle.pc_oracle import PCOracle
        kind = "port"
        kw = dict(HYPER)
        if w["kind"] == "full":
            kw.update(cross_entropy=True, optimizer="ADAM", psi_optimizer="ADAM")
        net = PCOracle(w["kind"], sizes, w["batch"], act=w["act"], **kw)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set(l, nm, v)
    run = (lambda: net.train_step_python(x, y, w["T"])) if (kind == "port" and w["kind"] == "simple") \
        else (lambda: net.train_step(x, y, w["T"]))
    return run, kind, sizes


def cpu_reference_leg(w, steps, warmup, seconds_wanted=25.0, sample_hidden=None):
    """The reference's CPU train step on a depth-reduced copy of the workload.

    The sample depth is picked from a calibration step on a 16-layer cut so that
    warmup + steps sample steps take about `seconds_wanted` seconds (capped at 256 layers), unless
    `sample_hidden` fixes it.  Threads: the reference's own DynamicThread policy first
    (include/deepity/utils/Optimize.h:108-131); if half the affinity mask is faster on this
    host (OpenMP plus OpenBLAS pools oversubscribing it), that count is used instead and both
    timings are reported.  Returns samples/s scaled to the full depth by the FLOP ratio."""
    from oracle import ref as oref
    host = host_cpu_info()
    full_hidden = w["hidden"]
    threads_policy = threads_used = None
    calib = {}
    deep = w["width"] >= 512 and full_hidden > 32
    if deep and oref.available():
        run16, _, sizes16 = _cpu_net(w, 16)
        run16()
        threads_policy = oref.host_info()["omp_threads"]
        t0 = time.perf_counter()
        run16()
        t_policy = time.perf_counter() - t0
        half = max(1, min(threads_policy, host["affinity_cpus"] // 2))
        oref.set_threads(half)
        run16()
        t0 = time.perf_counter()
        run16()
        t_half = time.perf_counter() - t0
        threads_used = half if t_half < t_policy else threads_policy
        oref.set_threads(threads_used)
        per_layer = min(t_half, t_policy) / 17.0
        calib = {"calibration_layers": 16, "ms_per_step_policy_threads": t_policy * 1e3,
                 "ms_per_step_half_affinity_threads": t_half * 1e3,
                 "ms_per_layer_at_16": per_layer * 1e3}
        if sample_hidden is None:
            want = seconds_wanted / ((steps + warmup) * per_layer)
            sample_hidden = 256 if want >= 256 else 128 if want >= 128 else 64 if want >= 64 else 32
    hidden = min(full_hidden, sample_hidden or (64 if deep else full_hidden))
    run, kind, sizes = _cpu_net(w, hidden)
    for _ in range(warmup):
        run()
    if kind == "reference":
        info = oref.host_info()
        if threads_used is None:
            threads_policy = threads_used = info["omp_threads"]
        cores, blas = int(threads_used), info["blas"]
    else:
        cores, blas = os.cpu_count(), "numpy"
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        e = run()
        times.append(time.perf_counter() - t0)
    dt_mean, dt_min, dt_med = sum(times) / len(times), min(times), statistics.median(times)
    sample_flops = algorithmic_flops(w["kind"], sizes, w["batch"], w["T"])
    scale = algorithmic_flops(w["kind"], sizes_of(w), w["batch"], w["T"]) / sample_flops
    sps = w["batch"] / (dt_mean * scale)
    sample = (f"{w['desc']} cut to {hidden} hidden layers ({steps} steps, mean {dt_mean * 1e3:.1f} "
              f"min {dt_min * 1e3:.1f} median {dt_med * 1e3:.1f} ms); scaled x{scale:.2f} to "
              f"{full_hidden} layers by algorithmic FLOPs" if hidden != full_hidden
              else f"{w['desc']} at full size, {steps} steps, mean {dt_mean * 1e3:.1f} ms")
    return {"value": sps, "unit": "samples/s", "cores": cores, "kind": kind, "sample": sample,
            "extrapolated": hidden != full_hidden, "sample_hidden_layers": hidden,
            "scale_to_full_depth": scale, "steps_run": steps, "warmup_run": warmup,
            "ms_per_step_sample": dt_mean * 1e3, "ms_per_step_sample_min": dt_min * 1e3,
            "ms_per_step_sample_median": dt_med * 1e3,
            "ms_per_layer_sample": dt_mean * 1e3 / (hidden + 1),
            "cpu_gflops": sample_flops / dt_mean / 1e9, "threads_reference_policy": threads_policy,
            "threads_used": cores, "blas": blas, "host": host, "last_energy": float(e), **calib}


CPU_KEYS = ("value", "unit", "cores", "kind", "sample", "extrapolated", "sample_hidden_layers",
            "scale_to_full_depth", "steps_run", "ms_per_step_sample", "ms_per_step_sample_min",
            "ms_per_step_sample_median", "ms_per_layer_sample", "ms_per_layer_at_16", "cpu_gflops",
            "threads_reference_policy", "threads_used", "blas", "host",
            "ms_per_step_policy_threads", "ms_per_step_half_affinity_threads")


def cpu_keys(leg):
    return {k: leg[k] for k in CPU_KEYS if k in leg}


# ------------------------------------------------------------------------------ conv (C5)
def conv_layers():
    c, h, w = C5["input_shape"]
    out = []
    for i, (o, kh, kw, sh, sw, ph, pw) in enumerate(C5["convs"]):
        out.append(dict(inC=c, outC=o, H=h, W=w, kH=kh, kW=kw, sH=sh, sW=sw, pH=ph, pW=pw,
                        act=C5["act"] if i + 1 < len(C5["convs"]) else "linear"))
        c, h, w = o, (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    out.append(dict(inC=c, outC=0, H=h, W=w, kH=1, kW=1, sH=1, sW=1, pH=0, pW=0, act="linear"))
    return out


def conv_synth(layers, B, seed=1234, wseed=99):
    rng, wr = np.random.default_rng(seed), np.random.default_rng(wseed)
    f = layers[0]
    x = rng.normal(size=(B, f["inC"], f["H"], f["W"])).astype(np.float32)
    y = np.eye(layers[-1]["inC"], dtype=np.float32)[rng.integers(0, layers[-1]["inC"], B)]
    params = []
    for d in layers[:-1]:
        rows = d["inC"] * d["kH"] * d["kW"]
        params.append(wr.normal(0, np.sqrt(2.0 / rows), (d["outC"], rows)).astype(np.float32))
    return x, y, params


def conv_flops(layers, B, T):
    """2*B*P*O*(C*kH*kW) per product: T+1 forward (the clamped input layer: 1), T transposed
    (none for the clamped input layer) and 1 weight-shaped product per weight layer."""
    total = 0.0
    for i, d in enumerate(layers[:-1]):
        oh = (d["H"] + 2 * d["pH"] - d["kH"]) // d["sH"] + 1
        ow = (d["W"] + 2 * d["pW"] - d["kW"]) // d["sW"] + 1
        g = 2.0 * B * oh * ow * d["outC"] * d["inC"] * d["kH"] * d["kW"]
        total += g * ((1 if i == 0 else T + 1) + (0 if i == 0 else T) + 1)
    return total


def conv_cpu_leg(layers, B, T, steps, warmup):
    from oracle import ref as oref
    x, y, params = conv_synth(layers, B)
    if oref.available():
        kind, cores = "reference", oref.host_info()["omp_threads"]
        net = oref.RefConvNet(layers, B, HYPER["lr"], HYPER["ir"], HYPER["lmbda"])
    else:
        from oracle.conv_oracle import ConvOracle
        kind, cores = "port", os.cpu_count()
        net = ConvOracle(layers, B, HYPER["lr"], HYPER["ir"], HYPER["lmbda"])
    for l, W in enumerate(params):
        net.set(l, "W", W)
    for _ in range(warmup):
        net.train_step(x, y, T)
    t0 = time.perf_counter()
    for _ in range(steps):
        e = net.train_step(x, y, T)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"value": B / dt, "unit": "samples/s", "cores": int(cores), "kind": kind,
            "sample": f"{C5['desc']} at full size, {steps} steps of {dt * 1e3:.1f} ms",
            "last_energy": float(e)}


def conv_main(args):
    """--workload c5: the convolutional network on one GPU (replicas only beyond that)."""
    layers, B, T = conv_layers(), C5["batch"], C5["T"]
    config = {"workload": C5["desc"], "global_batch": B, "T": T, "layers": len(layers) - 1,
              "hyper": {k: HYPER[k] for k in ("lr", "ir", "lmbda")}, "precision": "fp32",
              "l2": "L2 flushed between timed steps"}
    if args.impl == "reference":
        leg = conv_cpu_leg(layers, B, T, max(1, args.steps), max(1, args.warmup))
        print(json.dumps({"impl": "reference", "metric": "train_step samples/sec",
                          "value": leg["value"], "unit": "samples/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": B / leg["value"] * 1e3, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic", "config": config,
                          "cpu_baseline": {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")},
                          "e2e": {"value": leg["value"], "unit": "samples/s",
                                  "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    import torch
    import deepity_b200 as dp
    from deepity_b200 import _lib
    torch.cuda.set_device(0)
    lib = _lib.load()
    arch = []
    for d in layers:
        arch.append(dp.Convolution(d["outC"], d["kH"], d["kW"], d["sH"], d["sW"], d["pH"], d["pW"]))
        if d["act"] != "linear":
            arch.append(dp.ReLU())
    net = dp.SimpleConvolutionalPCN(*arch, input_shape=C5["input_shape"], batch_size=B)
    net.configure(learning_rate=HYPER["lr"], inference_rate=HYPER["ir"], lmbda=HYPER["lmbda"], seed=1)
    x, y, params = conv_synth(layers, B)
    for l, W in enumerate(params):
        net.set_tensor(l, "W", W)
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    ctx = lib.dpcn_conv_context(net._h)
    stream = torch.cuda.ExternalStream(lib.dpc_stream(ctx))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def timed(fn, steps):
        total = 0.0
        for _ in range(steps):
            flush.zero_()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            b.synchronize()
            total += a.elapsed_time(b)
        return total / steps

    for _ in range(args.warmup):
        energy = net.train_step_device(xd, yd, T)
    with ClockSampler(0) as clk:
        n0 = net.launch_count
        ms = timed(lambda: net.train_step_device(xd, yd, T), args.steps)
        launches = net.launch_count - n0
        energy = net.train_step_device(xd, yd, T)
        e2e_ms = timed(lambda: net.train_step(x, y, T), args.steps)
        # dominant kernel: the forward implicit GEMM of the widest layer (64 -> 128 channels)
        plan, big = lib.dpcn_conv_plan(net._h), 2
        for _ in range(2):
            lib.dpc_conv_forward(plan, big, 2)
        k_ms = timed(lambda: lib.dpc_conv_forward(plan, big, 2), max(args.steps, 5))
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    d = layers[big]
    oh, ow = layers[big + 1]["H"], layers[big + 1]["W"]
    rows = d["inC"] * d["kH"] * d["kW"]
    k_flops = 2.0 * B * oh * ow * d["outC"] * rows
    k_bytes = 4.0 * (B * d["inC"] * d["H"] * d["W"] + d["outC"] * rows + 5 * B * d["outC"] * oh * ow)
    hbm = peaks.get("hbm_gbs") or 6650.0
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    flops = conv_flops(layers, B, T)
    line = {"metric": "train_step samples/sec", "value": B / (ms * 1e-3), "unit": "samples/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config, "energy": energy,
            "algorithmic_flops_per_step": flops, "achieved_tflops_step": flops / (ms * 1e-3) / 1e12,
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(x.nbytes + y.nbytes), "d2h_bytes_per_step": 8},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "conv forward implicit GEMM, 64->128 channels "
                                                   "(reads z, W, z_up; writes preact, mu, e_up, g)",
                         "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                         "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback",
                         "traffic": None, "launch_ms": k_ms, "algorithmic_bytes_per_launch": k_bytes,
                         "algorithmic_flops_per_launch": k_flops,
                         "note": "7.6 MB and 0.3 GFLOP per launch on 64 CTAs: latency-bound at this size, "
                                 "neither roofline binds"},
            "clocks": clk.summary()}
    if not args.no_cpu:
        leg = conv_cpu_leg(layers, B, T, 2, 1)
        line["cpu_baseline"] = {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))


# ------------------------------------------------------------------------------ GPU leg
def build_net(w, sizes, precision):
    import deepity_b200 as dp
    acts = {"tanh": dp.TanH, "sigmoid": dp.Sigmoid, "gelu": dp.GeLU, "relu": dp.ReLU}
    arch = []
    for l in range(len(sizes) - 1):
        arch.append(dp.Linear(sizes[l], sizes[l + 1]))
        arch.append(acts[w["act"]]())
    cls = {"dkp": dp.DKPPCN, "simple": dp.SimplePCN, "full": dp.FullPCN}[w["kind"]]
    net = cls(*arch, batch_size=w["batch"], device=f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}")
    kw = dict(learning_rate=HYPER["lr"], inference_rate=HYPER["ir"], lmbda=HYPER["lmbda"], seed=1,
              precision=precision)
    if w["kind"] != "simple":
        kw.update(feedback_rate=HYPER["fl"])
    if w["kind"] == "full":
        kw.update(use_cross_entropy=True, optimizer="ADAM", psi_optimizer="ADAM")
    net.configure(**kw)
    return net


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


# DRAM bytes per 1024x512x512 layer of one launch of the dominant kernel, measured with ncu
# (dram__bytes_read.sum + dram__bytes_write.sum) as the difference between a 127-layer and a
# 63-layer capture divided by 64, so that the dirty lines a launch leaves in L2 cancel:
# (669.2 + 478.8) MB - (333.0 + 214.7) MB = 600.3 MB over 64 layers (algorithmic: 9.44 MB).
NCU_DRAM_BYTES_PER_LAYER = 9.38e6


def forward_roofline(B, sizes, k_ms, precision, passes, peaks):
    """Roofline object of the grouped forward GEMM of a settling pass (layers 1..n-2).

    Both floors are stated: tensor time = passes x algorithmic FLOPs / measured dense bf16
    burst peak (a TF32 pass counts twice: half the bf16 rate), HBM time = algorithmic bytes /
    measured copy bandwidth.  `bound` is the larger floor; achieved/peak/frac follow it."""
    n = len(sizes)
    k_flops = sum(2.0 * B * sizes[i] * sizes[i + 1] for i in range(1, n - 1))
    # per layer: read z and W (operands), z of the layer above; write e of the layer above, fe
    k_bytes = sum(4.0 * (B * sizes[i] + sizes[i] * sizes[i + 1] + 3 * B * sizes[i + 1])
                  for i in range(1, n - 1))
    peak_tf = peaks.get("bf16_tflops") or 1590.0
    hbm = peaks.get("hbm_gbs") or 6650.0
    src = "measured (MEASURED_PEAKS.json)" if peaks else "fallback (6.65 TB/s, 1.59 PFLOP/s)"
    t = k_ms * 1e-3
    tflops, gbs = k_flops / t / 1e12, k_bytes / t / 1e9
    tensor_floor_ms = passes * k_flops / (peak_tf * 1e12) * 1e3
    hbm_floor_ms = k_bytes / (hbm * 1e9) * 1e3
    bound = "hbm" if hbm_floor_ms >= tensor_floor_ms else "tensor"
    r = {"bound": bound,
         "achieved": gbs if bound == "hbm" else tflops,
         "peak": hbm if bound == "hbm" else peak_tf,
         "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
         "frac": gbs / hbm if bound == "hbm" else tflops / peak_tf,
         "peak_source": src + (": hbm_gbs" if bound == "hbm" else ": bf16_tflops (burst; kernel timed alone)"),
         "traffic": (NCU_DRAM_BYTES_PER_LAYER * (n - 2)
                     if NCU_DRAM_BYTES_PER_LAYER and (B, sizes[1]) == (1024, 512) else None),
         "kernel": "grouped forward GEMM of a settling pass + bias/activation/error/feedback-error "
                   "epilogue (pc_tc_kernel<0,256,...> CTA pairs)",
         "launch_ms": k_ms, "layers_per_launch": n - 2,
         "algorithmic_flops_per_launch": k_flops, "algorithmic_bytes_per_launch": k_bytes,
         "tensor_passes": passes,
         "tflops_at_algorithmic_flops": tflops, "frac_of_bf16_peak": tflops / peak_tf,
         "frac_of_bf16_peak_counting_passes": passes * tflops / peak_tf,
         "hbm_gbs_at_algorithmic_bytes": gbs, "frac_of_hbm_peak": gbs / hbm,
         "tensor_floor_ms": tensor_floor_ms, "hbm_floor_ms": hbm_floor_ms,
         "frac_of_binding_floor": max(tensor_floor_ms, hbm_floor_ms) / k_ms}
    return r


def plan_paths(lib, net, n_layers):
    """Which kernels a plan runs: the tensor-core run and what falls to the CUDA cores."""
    import ctypes
    first, count = ctypes.c_int(), ctypes.c_int()
    plan = lib.dpcn_plan(net._h)
    lib.dpc_plan_tensor_run(plan, ctypes.byref(first), ctypes.byref(count))
    buf = ctypes.create_string_buffer(256)
    lib.dpc_plan_describe(plan, buf, 256)
    return {"tensor_core_layers": [first.value, first.value + count.value],
            "cuda_core_weight_layers": (n_layers - 1) - count.value,
            "kernels": buf.value.decode()}


def dist_setup():
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def timed_ranks(fn, steps, stream):
    """K calls bracketed by barrier + synchronize, CUDA events on `stream`, max over ranks."""
    import torch
    import torch.distributed as dist
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(steps):
        fn()
    b.record(stream)
    b.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def layer_sharded_main(args, w, sizes, config):
    """The N>1 arm: layer-sharded deep stack, strong scaling (the same network and batch at
    every N), timed on the device with CUDA events, max over ranks."""
    import torch
    import torch.distributed as dist
    from deepity_b200.sharded import ShardedDKPPCN

    rank, world, local = dist_setup()
    net = ShardedDKPPCN(sizes, w["batch"], HYPER, act=w["act"], precision=args.precision)
    x, y, params = synth(w, sizes)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_param(l, nm, v)
    del params
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    xh, yh = torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()
    T, B = w["T"], w["batch"]
    for _ in range(args.warmup):
        energy = net.train_step(xd, yd, T)
    with ClockSampler(local) as clk:
        n0 = net.eng.launch_count
        ms = timed_ranks(lambda: net.train_step(xd, yd, T, read_energy=False), args.steps,
                         net.eng.stream)
        launches = net.eng.launch_count - n0
        energy = net.train_step(xd, yd, T)
        for _ in range(2):  # untimed: first host-buffer steps (pinned staging, NCCL set-up)
            net.train_step(xh, yh, T)
        e2e_ms = timed_ranks(lambda: net.train_step(xh, yh, T), args.steps, net.eng.stream)
    lc = torch.tensor([launches], device="cuda", dtype=torch.int64)
    dist.all_reduce(lc)
    flops = net.train_step_flops(T)
    ranges = net.ranges
    # dominant kernel on this rank's block of layers (the same settle-pass forward launch as at
    # N = 1, over the local layers), timed alone with CUDA events on the library's stream; the
    # slowest rank's figure is reported
    eng = net.eng
    local_sizes = list(eng.sizes)
    k_first, k_count = 1, len(local_sizes) - 2
    fwd_flags = 2 | 8 | 256  # DPC_FWD_ERR_NEXT | DPC_FWD_FE | DPC_FWD_TRANSIENT
    k_ms = None
    if k_count > 0:
        for _ in range(3):
            eng.lib.dpc_forward(eng.plan, k_first, k_count, fwd_flags)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(args.steps, 5)
        a.record(eng.stream)
        for _ in range(reps):
            eng.lib.dpc_forward(eng.plan, k_first, k_count, fwd_flags)
        b.record(eng.stream)
        b.synchronize()
        k_ms = a.elapsed_time(b) / reps
    kt = torch.tensor([k_ms or 0.0, float(k_count)], device="cuda", dtype=torch.float64)
    gathered = [torch.zeros_like(kt) for _ in range(world)]
    dist.all_gather(gathered, kt)
    # (the sharded network stays alive to the end of the process: torch tensors that were used on
    # its stream outlive this function, and freeing them after the stream is gone aborts)
    side = None if args.no_side else batch_sharded_measure(args, dict(WORKLOADS["c4"]))
    if rank == 0:
        peaks = load_peaks()
        peak = (peaks.get("bf16_tflops_sustained") or 1590.0) * world
        config = dict(config, parallelism=f"layer-sharded x{world}",
                      layers_per_rank=[e - b for b, e in ranges])
        # per-layer time of the slowest rank's launch -> the roofline object of that launch
        per_rank = [(float(g[0]), int(g[1])) for g in gathered]
        slow_ms, slow_layers = max(per_rank, key=lambda t: t[0] / max(t[1], 1))
        roofline = None
        if slow_layers > 0:
            H = sizes[1]
            roofline = forward_roofline(B, [H] * (slow_layers + 2), slow_ms, args.precision,
                                        2 if args.precision == "tf32" else 3, peaks)
            roofline["per_rank_launch_ms"] = [round(t[0], 4) for t in per_rank]
            roofline["per_rank_layers"] = [t[1] for t in per_rank]
        line = {"metric": "train_step samples/sec", "value": B / (ms * 1e-3), "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": DTYPES[args.precision], "data": "synthetic",
                "config": config, "energy": energy, "algorithmic_flops_per_step": flops,
                "achieved_tflops_step": flops / (ms * 1e-3) / 1e12,
                "frac_of_gemm_peak_step": flops / (ms * 1e-3) / 1e12 / peak,
                "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": int(x.nbytes + y.nbytes), "d2h_bytes_per_step": 8},
                "gpu_launches": int(lc.item()), "clocks": clk.summary(),
                "roofline": roofline, "cpu_baseline": None, "batch_sharded_c4": side}
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def batch_sharded_measure(args, w, steps=None):
    """The wide FullPCN workload batch-sharded over the ranks of the job (strong scaling: the
    same network and GLOBAL batch at every N); returns the measurement on every rank."""
    import torch
    import torch.distributed as dist
    from deepity_b200.sharded import BatchSharded

    rank, world, local = dist_setup()
    sizes = sizes_of(w)
    x, y, params = synth(w, sizes)
    T, B = w["T"], w["batch"]
    steps = steps or max(3, min(args.steps, 10))

    def build(local_batch):
        net = build_net(dict(w, batch=local_batch), sizes, args.precision)
        for l, p in enumerate(params):
            for nm, v in p.items():
                net.set_tensor(l, nm, v)
        return net
    net = BatchSharded(build, B)
    lib = net.net._lib
    stream = torch.cuda.ExternalStream(lib.dpc_stream(lib.dpcn_context(net.net._h)))
    xd = torch.from_numpy(np.ascontiguousarray(net.rows(x))).cuda()
    yd = torch.from_numpy(np.ascontiguousarray(net.rows(y))).cuda()
    for _ in range(max(2, min(args.warmup, 3))):
        energy = net.train_step_device(xd, yd, T)
    n0 = net.net.launch_count
    ms = timed_ranks(lambda: net.train_step_device(xd, yd, T, read_energy=False), steps, stream)
    launches = net.net.launch_count - n0
    energy = net.train_step_device(xd, yd, T)
    for _ in range(2):
        net.train_step(x, y, T)
    e2e_ms = timed_ranks(lambda: net.train_step(x, y, T), steps, stream)
    lc = torch.tensor([launches], device="cuda", dtype=torch.int64)
    dist.all_reduce(lc)
    flops = algorithmic_flops(w["kind"], sizes, B, T)
    return {"workload": w["desc"], "parallelism": f"batch-sharded x{world}",
            "rows_per_rank": B // world, "value": B / (ms * 1e-3), "unit": "samples/s",
            "ms_per_step": ms, "steps": steps, "scaling": "strong", "energy": energy,
            "algorithmic_flops_per_step": flops, "achieved_tflops_step": flops / (ms * 1e-3) / 1e12,
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int((x.nbytes + y.nbytes) // world),
                    "d2h_bytes_per_step": 8},
            "gpu_launches": int(lc.item())}


def batch_sharded_main(args, w, sizes, config):
    """--workload c4 at N>1: the batch-sharded measurement as the headline of the line."""
    import torch.distributed as dist
    rank, world, local = dist_setup()
    with ClockSampler(local) as clk:
        m = batch_sharded_measure(args, w, steps=args.steps)
    if rank == 0:
        config = dict(config, parallelism=m["parallelism"], rows_per_rank=m["rows_per_rank"])
        line = {"metric": "train_step samples/sec", "value": m["value"], "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": DTYPES[args.precision], "data": "synthetic",
                "config": config, "energy": m["energy"],
                "algorithmic_flops_per_step": m["algorithmic_flops_per_step"],
                "achieved_tflops_step": m["achieved_tflops_step"], "e2e": m["e2e"],
                "gpu_launches": m["gpu_launches"], "clocks": clk.summary(),
                "roofline": None, "cpu_baseline": None}
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


DTYPES = {"fp32": "f32 (tensor-core layers: 3xBF16 operand split for SGD networks, 3xTF32 otherwise)",
          "tf32": "tf32", "mixed": "as f32 where the plan keeps operand planes; else f32 state path, tf32 gradient path"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["c5"])
    ap.add_argument("--depth", type=int, default=None, help="override the hidden-layer count")
    ap.add_argument("--precision", default="fp32", choices=["fp32", "tf32", "mixed"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-side", action="store_true",
                    help="skip the batch-sharded C4 measurement that rides along with C3")
    ap.add_argument("--sweep-trace", action="store_true",
                    help="print the per-layer time stamps of the forward-sweep kernel "
                         "(c3 cut to 300 hidden layers unless --depth is given) and exit")
    ap.add_argument("--sample-depth", type=int, default=None,
                    help="hidden layers of the CPU arm's bounded sample (default: calibrated)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.workload == "c5":
        if rank == 0:
            conv_main(args)
        return
    w = dict(WORKLOADS[args.workload])
    if args.depth:
        w["hidden"] = args.depth
        w["desc"] += f" (depth overridden to {args.depth})"
    sizes = sizes_of(w)
    B, T = w["batch"], w["T"]
    config = {"workload": w["desc"], "global_batch": B, "T": T, "layers": len(sizes) - 1,
              "hyper": HYPER, "precision": args.precision,
              "parity_bound": "1e-4 relative per tensor for SGD networks; 5e-4 where an Adam-type "
                              "optimizer is on; 1e-2 in tf32 mode; 1e-3 in mixed mode",
              "l2": "working set (z,e,preact,mu,fe,W of every layer) is far larger than the 126 MB L2"
              if args.workload in ("c3", "c4") else "L2 flushed between timed steps"}

    if args.sweep_trace:
        if rank == 0:
            sweep_trace(args, w)
        return

    if args.impl == "reference":
        if rank != 0:
            return
        # K steps and W warm-up steps of a bounded sample (see the module docstring)
        leg = cpu_reference_leg(w, max(1, args.steps), max(1, args.warmup), seconds_wanted=90.0,
                                sample_hidden=args.sample_depth)
        line = {"impl": "reference", "metric": "train_step samples/sec", "value": leg["value"],
                "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": leg["ms_per_step_sample"],
                "ms_per_step_is": "one train step of the bounded sample (measured)",
                "extrapolated": leg["extrapolated"],
                "sample_hidden_layers": leg["sample_hidden_layers"],
                "scale_to_full_depth": leg["scale_to_full_depth"],
                "ms_per_step_full_depth_extrapolated": B / leg["value"] * 1e3,
                "cpu_gflops": leg["cpu_gflops"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": cpu_keys(leg),
                "e2e": {"value": leg["value"], "unit": "samples/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    from deepity_b200 import _lib

    if world > 1:
        # deep stacks shard by layers; wide, shallow networks by batch rows
        if w["kind"] == "dkp" and len(sizes) - 1 >= world:
            layer_sharded_main(args, w, sizes, config)
        else:
            batch_sharded_main(args, w, sizes, config)
        return

    torch.cuda.set_device(0)
    lib = _lib.load()
    net = build_net(w, sizes, args.precision)
    x, y, params = synth(w, sizes)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_tensor(l, nm, v)
    del params
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    xh, yh = x.ravel().copy(), y.ravel().copy()
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(lib.dpc_stream(lib.dpcn_context(net._h)))
    flush = None
    if args.workload in ("c1", "c2"):
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def timed(fn, steps):
        """Mean ms per step over `steps` calls, CUDA events on the library's stream."""
        total = 0.0
        for _ in range(steps):
            if flush is not None:
                flush.zero_()
                torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            b.synchronize()
            total += a.elapsed_time(b)
        return total / steps

    flops = net.train_step_flops(T)
    paths = plan_paths(lib, net, len(sizes))
    for _ in range(args.warmup):
        energy = net.train_step_device(xd, yd, T)
    lib.dpc_sync(lib.dpcn_context(net._h))
    with ClockSampler(0) as clk:
        n0 = net.launch_count
        ms = timed(lambda: net.train_step_device(xd, yd, T, read_energy=False), args.steps)
        launches = net.launch_count - n0
        energy = net.train_step_device(xd, yd, T)
        # end to end: host buffers in, energy out
        for _ in range(2):
            net.train_step(xh, yh, T)
        t0 = time.perf_counter()
        e2e_ms_ev = timed(lambda: net.train_step(xh, yh, T), args.steps)
        e2e_wall = (time.perf_counter() - t0) / args.steps * 1e3
        e2e_ms = max(e2e_ms_ev, e2e_wall) if flush is None else e2e_ms_ev
        # dominant kernel: the grouped forward GEMM of a settling pass (fused bias, activation,
        # error of the layer above and feedback error; predictions are not stored)
        plan = lib.dpcn_plan(net._h)
        n = len(sizes)
        fwd_flags = 2 | 8 | 256  # DPC_FWD_ERR_NEXT | DPC_FWD_FE | DPC_FWD_TRANSIENT
        for _ in range(3):
            lib.dpc_forward(plan, 1, n - 2, fwd_flags)
        k_ms = timed(lambda: lib.dpc_forward(plan, 1, n - 2, fwd_flags), max(args.steps, 5))
    clocks = clk.summary()

    peaks = load_peaks()
    peak_tf = peaks.get("bf16_tflops_sustained") or 1400.0
    # tensor passes per product: one TF32 pass = 2 bf16-rate passes; 3xBF16 = 3; 3xTF32 = 6
    sgd = w["kind"] != "full"
    passes = 2 if args.precision == "tf32" else (3 if sgd else 6)
    roofline = forward_roofline(B, sizes, k_ms, args.precision, passes, peaks)
    line = {"metric": "train_step samples/sec", "value": B / (ms * 1e-3), "unit": "samples/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPES[args.precision], "data": "synthetic",
            "config": config, "energy": energy, "paths": paths,
            "algorithmic_flops_per_step": flops, "achieved_tflops_step": flops / (ms * 1e-3) / 1e12,
            "frac_of_gemm_peak_step": flops / (ms * 1e-3) / 1e12 / peak_tf,
            "gemm_peak_step_source": "bf16_tflops_sustained (kernel timed inside a long step)",
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(xh.nbytes + yh.nbytes), "d2h_bytes_per_step": 8},
            "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks}
    if paths["cuda_core_weight_layers"] > 1 and args.workload in ("c3", "c4"):
        print(f"bench: {paths['cuda_core_weight_layers']} weight layers of this workload run on the "
              f"CUDA-core kernels ({paths['kernels']})", file=sys.stderr)
    if not args.no_cpu:
        leg = cpu_reference_leg(w, 5, 1, seconds_wanted=25.0, sample_hidden=args.sample_depth)
        line["cpu_baseline"] = cpu_keys(leg)
        if args.workload == "c3" and leg["kind"] == "reference":
            # the same cut on the GPU, same seeds and step count: the energies must agree
            line["cpu_baseline"]["energy_check"] = sample_energy_check(w, leg, args.precision)
    if args.workload == "c3" and not args.no_side and not args.depth:
        del net, xd, yd
        torch.cuda.empty_cache()
        line["c4_single_gpu"] = single_gpu_side(dict(WORKLOADS["c4"]), args)
    print(json.dumps(line))


def sample_energy_check(w, leg, precision):
    """Runs the CPU arm's sample (same cut, seeds and number of steps) on the GPU and reports
    the relative difference of the last step's energy."""
    hidden = leg["sample_hidden_layers"]
    sizes = sizes_of(w, hidden)
    net = build_net(w, sizes, precision)
    x, y, params = synth(w, sizes)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_tensor(l, nm, v)
    e = None
    for _ in range(leg["steps_run"] + leg["warmup_run"]):
        e = net.train_step(x, y, w["T"])
    ref = leg["last_energy"]
    return {"hidden_layers": hidden, "steps": leg["steps_run"] + leg["warmup_run"],
            "cpu_energy": ref, "gpu_energy": e, "relative_difference": abs(e - ref) / max(1.0, abs(ref))}


def sweep_trace(args, w):
    """Profiling aid: where a layer of the persistent forward-sweep kernel spends its time.
    CTA 0 of the kernel stamps %globaltimer at six points of every layer (the first 256 layers);
    prints the median differences over layers 50..250 as one JSON line."""
    import ctypes
    import torch
    from deepity_b200 import _lib
    if not args.depth:
        w = dict(w, hidden=300)
    sizes = sizes_of(w)
    torch.cuda.set_device(0)
    lib = _lib.load()
    net = build_net(w, sizes, args.precision)
    net.set_use_graph(False)
    stamps = torch.zeros(256 * 8, dtype=torch.int64, device="cuda")
    _lib.check(lib.dpc_plan_set_chain_trace(lib.dpcn_plan(net._h), ctypes.c_void_p(stamps.data_ptr())))
    x, y, params = synth(w, sizes)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_tensor(l, nm, v)
    for _ in range(3):
        net.train_step(x, y, w["T"])
    t = stamps.cpu().numpy().reshape(256, 8).astype(np.int64)
    _lib.check(lib.dpc_plan_set_chain_trace(lib.dpcn_plan(net._h), None))
    lo, hi = 50, min(250, len(sizes) - 4)
    d = t[lo:hi]
    med = lambda v: float(np.median(v))
    out = {"workload": w["desc"], "precision": args.precision, "hidden_layers": w["hidden"],
           "layers_sampled": [lo, hi], "unit": "ns (globaltimer, 32 ns steps)",
           "dependency_seen_to_first_operands_landed": med(d[:, 1] - d[:, 0]),
           "first_operands_to_accumulator_complete": med(d[:, 2] - d[:, 1]),
           "accumulator_complete_to_stores_issued": med(d[:, 3] - d[:, 2]),
           "of_which_until_partial_sums_exchanged": med(d[:, 5] - d[:, 2]),
           "stores_issued_to_published": med(d[:, 4] - d[:, 3]),
           "published_to_next_dependency_seen": med(t[lo + 1:hi + 1, 0] - d[:, 4]),
           "layer_period": med(t[lo + 1:hi + 1, 0] - d[:, 0])}
    print(json.dumps(out))


def single_gpu_side(w, args):
    """The wide FullPCN workload on one GPU (rides along with the headline line so that the
    batch-sharded figures of the multi-GPU lines have their N=1 point)."""
    import torch
    from deepity_b200 import _lib
    lib = _lib.load()
    sizes = sizes_of(w)
    net = build_net(w, sizes, args.precision)
    x, y, params = synth(w, sizes)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_tensor(l, nm, v)
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    stream = torch.cuda.ExternalStream(lib.dpc_stream(lib.dpcn_context(net._h)))
    T, B = w["T"], w["batch"]
    steps = max(3, min(args.steps, 10))
    for _ in range(3):
        energy = net.train_step_device(xd, yd, T)

    def timed(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        b.synchronize()
        return a.elapsed_time(b) / steps
    ms = timed(lambda: net.train_step_device(xd, yd, T, read_energy=False))
    energy = net.train_step_device(xd, yd, T)
    e2e_ms = timed(lambda: net.train_step(x, y, T))
    flops = net.train_step_flops(T)
    return {"workload": w["desc"], "value": B / (ms * 1e-3), "unit": "samples/s", "ms_per_step": ms,
            "steps": steps, "energy": energy, "algorithmic_flops_per_step": flops,
            "achieved_tflops_step": flops / (ms * 1e-3) / 1e12, "paths": plan_paths(lib, net, len(sizes)),
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(x.nbytes + y.nbytes), "d2h_bytes_per_step": 8}}


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the predictive-coding train step (metric: train_step samples/sec).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c2|c1|c4|c5] [--depth D] [--precision fp32|tf32|mixed]

One "step" is one full ``train_step`` (settle T times, learn, final energy) on one batch of
synthetic data.  At N=1 the workload is the configuration the headline metric is quoted on:
DKPPCN, width 512, 2048 hidden layers, batch 1024, T=2, tanh, SGD for W and Psi, inputs
N(0,1), one-hot 10-class targets (it fits one GPU: about 23 GB).  Printed on rank 0: ONE
JSON line with

* ``value``     samples/s with x,y already resident in HBM (``train_step_device``), timed with
                CUDA events on the library's own stream, max over ranks;
* ``e2e``       the same metric through the public host-buffer call ``net.train_step(x, y, T)``
                (pinned staging + H2D of x,y and the D2H energy read inside the timed region);
* ``roofline``  the dominant kernel (the grouped forward GEMM of one settling pass) timed on
                its own: algorithmic FLOPs per launch / mean launch time against the measured
                dense tensor peak of MEASURED_PEAKS.json;
* ``cpu_baseline`` the reference's own CPU code (oracle/_ref; numpy restatement if that is
                absent) on a bounded sample of the workload — the same network cut to a few
                layers, scaled to the full depth by the layer ratio;
* clocks sampled with nvidia-smi during the timed region.

``--impl reference`` times only the CPU leg, with the threads the reference's own policy
picks, and prints the same line shape with ``"impl": "reference"``.
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


def algorithmic_flops(kind, sizes, B, T):
    """GEMM FLOPs one train step needs under the reference's CPU semantics (2*M*N*K each):
    per weight layer T+3 (DirectKP), T+4 (Full) or T+1 (Simple) forward products, T feedback
    products and the weight-shaped products (learn, plus the direct-feedback update when the
    layer above owns feedback weights), plus the skinny Psi / projection products; the clamped
    input layer evaluates its prediction once and is never updated."""
    n = len(sizes)
    total = 0.0
    for i in range(n - 1):
        s, nx, ts = sizes[i], sizes[i + 1], sizes[-1]
        g = 2.0 * B * s * nx
        if kind == "simple":
            fwd, fb, wg = T + 1, T, 1
        else:
            fwd, fb, wg = (T + 3 if kind == "dkp" else T + 4), T, (2 if i + 2 < n else 1)
            total += 2.0 * B * s * ts + (2.0 * B * nx * ts if i + 2 < n else 0.0)
        if i == 0:
            fwd, fb = 1, 0
        total += g * (fwd + fb + wg)
    return total


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.index = index
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip().split(",")
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
                for nm, v in zip(names, out[2:]):
                    if v.strip().lower().startswith("active"):
                        self.reasons.add(nm)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------ CPU leg
def cpu_reference_leg(w, steps, warmup, budget_layers=None):
    """The reference's CPU train step on a depth-reduced copy of the workload.

    Returns dict(value=samples/s scaled to the full depth, cores, kind, sample)."""
    from oracle import ref as oref
    full_hidden = w["hidden"]
    hidden = min(full_hidden, budget_layers or (64 if w["width"] >= 512 else full_hidden))
    sizes = sizes_of(w, hidden)
    x, y, params = synth(w, sizes)
    opts = {}
    if w["kind"] == "full":
        opts = dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM")
    if oref.available():
        kind = "reference"
        net = oref.RefNet(w["kind"], sizes, w["batch"], act=w["act"], options=opts, **HYPER)
        info = oref.host_info()
        cores = info["omp_threads"]
    else:
        from oracle.pc_oracle import PCOracle
        kind = "port"
        kw = dict(HYPER)
        if w["kind"] == "full":
            kw.update(cross_entropy=True, optimizer="ADAM", psi_optimizer="ADAM")
        net = PCOracle(w["kind"], sizes, w["batch"], act=w["act"], **kw)
        cores = os.cpu_count()
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set(l, nm, v)
    run = (lambda: net.train_step_python(x, y, w["T"])) if (kind == "port" and w["kind"] == "simple") \
        else (lambda: net.train_step(x, y, w["T"]))
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        e = run()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    # Scale the sample's time to the full depth by the ratio of algorithmic FLOPs.
    scale = (algorithmic_flops(w["kind"], sizes_of(w), w["batch"], w["T"]) /
             algorithmic_flops(w["kind"], sizes, w["batch"], w["T"]))
    sps = w["batch"] / (dt * scale)
    sample = (f"{w['desc']} cut to {hidden} hidden layers ({steps} steps of {dt * 1e3:.1f} ms); "
              f"scaled x{scale:.2f} to {full_hidden} layers" if hidden != full_hidden
              else f"{w['desc']} at full size, {steps} steps of {dt * 1e3:.1f} ms")
    return {"value": sps, "unit": "samples/s", "cores": int(cores), "kind": kind,
            "sample": sample, "ms_per_step_sample": dt * 1e3, "last_energy": float(e)}


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
        leg = conv_cpu_leg(layers, B, T, max(1, min(args.steps, 3)), min(args.warmup, 1))
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
              "l2": "working set (z,e,preact,mu,fe,W of every layer) is far larger than the 126 MB L2"
              if args.workload in ("c3", "c4") else "L2 flushed between timed steps"}

    if args.impl == "reference":
        if rank != 0:
            return
        leg = cpu_reference_leg(w, max(1, min(args.steps, 3)), min(args.warmup, 1))
        line = {"impl": "reference", "metric": "train_step samples/sec", "value": leg["value"],
                "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": B / leg["value"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": leg["value"], "unit": "samples/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from deepity_b200 import _lib

    if world > 1:
        from deepity_b200 import sharded
        # deep stacks shard by layers; wide, shallow networks by batch rows
        if w["kind"] == "dkp" and len(sizes) - 1 >= world:
            sharded.bench_main(args, w, sizes, config)
        else:
            sharded.batch_bench_main(args, w, sizes, config)
        return

    torch.cuda.set_device(0)
    lib = _lib.load()
    net = build_net(w, sizes, args.precision)
    x, y, params = synth(w, sizes)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_tensor(l, nm, v)
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
        for _ in range(2):
            lib.dpc_forward(plan, 1, n - 2, fwd_flags)
        k_ms = timed(lambda: lib.dpc_forward(plan, 1, n - 2, fwd_flags), max(args.steps, 5))
    clocks = clk.summary()

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_tf = peaks.get("bf16_tflops_sustained") or 1590.0
    peak_src = "measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if peaks else "fallback 1.59 PF"
    hbm_peak = peaks.get("hbm_gbs") or 6650.0
    # per layer: read z, W and z of the layer above, write e of the layer above and fe
    k_flops = sum(2.0 * B * sizes[i] * sizes[i + 1] for i in range(1, n - 1))
    k_bytes = sum(4.0 * (B * sizes[i] + sizes[i] * sizes[i + 1] + 3 * B * sizes[i + 1])
                  for i in range(1, n - 1))
    tflops = k_flops / (k_ms * 1e-3) / 1e12
    gbs = k_bytes / (k_ms * 1e-3) / 1e9
    # ncu (profiles/pc_tc_kernel_forward_ncu.md): 438.7 MB of DRAM traffic for the 63 layers of
    # the captured small case = 6.96 MB per 1024x512x512 layer; it grows with the layer count
    traffic = 6.96e6 * (n - 2) if (w["batch"], w["width"]) == (1024, 512) else None
    if args.precision == "tf32":
        # one TF32 pass: 57 FLOP per algorithmic byte, below the machine balance -> HBM-bound
        roofline = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                    "frac": gbs / hbm_peak,
                    "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback"}
    else:
        # fp32 mode: three tensor passes per product (3xBF16 on SGD networks, else 3xTF32) ->
        # tensor-bound; the denominator is the measured bf16 peak, of which fp32-accurate
        # arithmetic can reach at most 1/3 (3xBF16) or 1/6 (3xTF32)
        roofline = {"bound": "tensor", "achieved": tflops, "peak": peak_tf, "unit": "TFLOP/s",
                    "frac": tflops / peak_tf, "peak_source": peak_src}
    roofline.update({"kernel": "grouped forward GEMM of a settling pass + error + feedback-error "
                               "epilogue (pc_tc_kernel<0,256,*,128,1>)",
                     "traffic": traffic, "launch_ms": k_ms,
                     "algorithmic_flops_per_launch": k_flops,
                     "algorithmic_bytes_per_launch": k_bytes,
                     "tflops_at_algorithmic_flops": tflops, "tensor_peak_tflops_bf16": peak_tf,
                     "hbm_gbs_at_algorithmic_bytes": gbs, "hbm_peak_gbs": hbm_peak})
    line = {"metric": "train_step samples/sec", "value": B / (ms * 1e-3), "unit": "samples/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"fp32": "f32", "tf32": "tf32", "mixed": "f32 state path, tf32 gradient path"}[
                args.precision], "data": "synthetic",
            "config": config, "energy": energy,
            "algorithmic_flops_per_step": flops, "achieved_tflops_step": flops / (ms * 1e-3) / 1e12,
            "frac_of_gemm_peak_step": flops / (ms * 1e-3) / 1e12 / peak_tf,
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(xh.nbytes + yh.nbytes), "d2h_bytes_per_step": 8},
            "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks}
    if not args.no_cpu:
        leg = cpu_reference_leg(w, 2, 1)
        line["cpu_baseline"] = {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))


if __name__ == "__main__":
    main()

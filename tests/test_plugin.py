"""The drop-in plugin boundary: libDeepityCUDA.so exports exactly the factory the reference's
loader resolves (src/backend/cuda/CUDAPluginExports.cpp:12-21,
src/backend/CUDAPluginLoader.cpp:52-107), and an UNMODIFIED reference network built with
DEVICE_GPU -- the compiled reference host of oracle/_ref, whose loader dlopens the plugin from
its own directory -- trains on this repository's kernels and agrees with the reference's CPU
backend at the reference's own CPU-vs-GPU bound of 1e-2
(tests/tDirectKPBatchedGPUVerify.cpp:47-58 in the reference)."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from common import make_case

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "deepity_b200", "libDeepityCUDA.so")
BESIDE_HOST = os.path.join(ROOT, "oracle", "_ref", "libDeepityCUDA.so")
GPU_VS_CPU = 1e-2


@pytest.fixture(scope="module")
def plugin_beside_host():
    """The loader looks next to the host module: put the plugin there (as the reference's build
    installs DeepityCUDA next to its extension module)."""
    from oracle import ref
    if not os.path.exists(PLUGIN):
        from deepity_b200 import build
        if build.build_plugin() is None:
            pytest.skip("libDeepityCUDA.so is not built and the reference checkout is absent")
    if not ref.available():
        pytest.skip("the compiled reference host (oracle/_ref) is not present")
    if os.path.lexists(BESIDE_HOST):
        os.remove(BESIDE_HOST)
    shutil.copy2(PLUGIN, BESIDE_HOST)
    return BESIDE_HOST


def test_plugin_exports_only_the_factory():
    if not os.path.exists(PLUGIN):
        pytest.skip("libDeepityCUDA.so is not built")
    out = subprocess.run(["nm", "-D", "--defined-only", PLUGIN], capture_output=True, text=True).stdout
    exported = [line.split()[-1] for line in out.splitlines() if " T " in line]
    assert exported == ["Deepity_CreateCUDABackend"], exported


def test_without_a_device_the_plugin_fails_loudly(plugin_beside_host):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from oracle import ref
    # the loader finds the plugin, the plugin's constructor refuses to run without a GPU
    with pytest.raises(RuntimeError):
        ref.RefNet("dkp", [8, 8, 4], 4, device="gpu")


def _run(kind, sizes, batch, T, steps, device, hyper, options=None, seed=0):
    from oracle import ref
    params, x, y = make_case(kind, sizes, batch, seed=seed)
    h = dict(hyper)
    if kind == "simple":
        h["fl"] = 0.0
    net = ref.RefNet(kind, sizes, batch, options=options or {}, device=device, **h)
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set(l, name, v)
    out = {"energies": np.asarray([net.train_step(x, y, T) for _ in range(steps)])}
    names = ["z", "e", "W", "b"] + ([] if kind == "simple" else ["Psi"])
    for l in range(net.num_layers):
        for name in names:
            a = net.get(l, name)
            if a.size:
                out[f"{l}.{name}"] = a
    out["predict"] = net.predict(x, T, with_projection=(kind != "simple"))
    return out


def _compare(cpu, gpu, what):
    worst = 0.0
    for k, r in cpu.items():
        r, g = np.asarray(r, dtype=np.float64), np.asarray(gpu[k], dtype=np.float64)
        assert r.shape == g.shape, (k, r.shape, g.shape)
        err = float(np.max(np.abs(r - g) / np.maximum(1.0, np.abs(r)))) if k == "energies" else \
            float(np.abs(r - g).max() / max(1.0, np.abs(r).max()))
        worst = max(worst, err)
        assert err <= GPU_VS_CPU, (what, k, err)
    print(f"{what}: reference network on the plugin vs on its CPU backend, worst error {worst:.2e}")
    return worst


CASES = {
    # below the tile sizes of the tensor-core GEMM: every product on the fp32 CUDA-core kernel
    "dkp_small": dict(kind="dkp", sizes=[32, 64, 64, 64, 10], batch=32, T=2, steps=3,
                      hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    # the reference's batched-run path (>= 4 layers of one width) at shapes the tcgen05 GEMM takes
    "dkp_batched_run_tensor_cores": dict(kind="dkp", sizes=[256] * 7 + [10], batch=256, T=2, steps=3,
                                         hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "full_ce_adam": dict(kind="full", sizes=[30, 40, 40, 10], batch=16, T=4, steps=3,
                         hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="gelu"),
                         options=dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM")),
    "simple_sigmoid": dict(kind="simple", sizes=[40, 24, 24, 10], batch=8, T=6, steps=3,
                           hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="sigmoid")),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_network_runs_on_the_plugin(name, plugin_beside_host):
    case = CASES[name]
    args = (case["kind"], case["sizes"], case["batch"], case["T"], case["steps"])
    cpu = _run(*args, "cpu", case["hyper"], case.get("options"))
    gpu = _run(*args, "gpu", case["hyper"], case.get("options"))
    _compare(cpu, gpu, name)

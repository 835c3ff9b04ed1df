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
    # what the reference's own CPU-vs-GPU test compares (tests/tDirectKPBatchedGPUVerify.cpp:
    # 127-262): energies, trained parameters and a prediction.  Its GPU path is allowed to leave
    # different transient states behind than its CPU path (it refreshes the clamped layer's
    # prediction where the CPU path keeps the cached one), so z and e are not compared.
    names = ["W", "b"] + ([] if kind == "simple" else ["Psi"])
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
    # shapes the tcgen05 GEMM takes (multiples of 128 / 64 / 32), every product of the step on the
    # tensor cores in one TF32 pass.  Widths alternate so that the reference's batched-run path
    # (>= 2 consecutive uniform layers on the GPU) stays out: that path fills the run's beliefs
    # from ONE batched product over stale inputs (src/networks/DirectKPPCNetwork.cpp:119-133)
    # where its CPU path sweeps layer by layer, so the reference's own two paths differ on runs
    # longer than two layers whatever backend executes them (dkp_small has a run of two).
    "dkp_tensor_core_shapes": dict(kind="dkp", sizes=[256, 512, 256, 512, 10], batch=256, T=2,
                                   steps=3,
                                   hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "full_ce_adam": dict(kind="full", sizes=[30, 40, 40, 10], batch=16, T=4, steps=3,
                         hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="gelu"),
                         options=dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM")),
    "simple_sigmoid": dict(kind="simple", sizes=[40, 24, 24, 10], batch=8, T=6, steps=3,
                           hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="sigmoid")),
}


GEMM_SHAPES = [
    # (M, N, K): tile-aligned shapes go to the tcgen05 kernel, the others to the CUDA-core kernel
    (256, 256, 256), (256, 128, 256), (128, 64, 32), (384, 192, 96),
    (100, 37, 53), (1, 10, 256), (256, 10, 128), (64, 64, 64),
]


@pytest.mark.gpu
@pytest.mark.parametrize("shape", GEMM_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_plugin_matmul_matches_blas(shape, plugin_beside_host):
    """IComputeBackend::MatMul of the plugin against numpy for every transposition, alpha/beta and
    padded leading dimensions: TF32 (the default, as on the reference's GPU backend) within 2e-3
    of the product's scale, and after SetAllowTF32(false) within fp32 rounding."""
    from oracle import ref
    M, N, K = shape
    rng = np.random.default_rng(M * 1000 + N * 10 + K)
    for ta in (False, True):
        for tb in (False, True):
            pad = 4 if (M % 4 == 0 and N % 4 == 0 and K % 4 == 0) else 3
            a_rows, a_cols = (K, M) if ta else (M, K)
            b_rows, b_cols = (N, K) if tb else (K, N)
            lda, ldb, ldc = a_cols + pad, b_cols + pad, N + pad
            A = rng.normal(size=(a_rows, lda)).astype(np.float32)
            B = rng.normal(size=(b_rows, ldb)).astype(np.float32)
            C0 = rng.normal(size=(M, ldc)).astype(np.float32)
            opA = A[:, :a_cols].T if ta else A[:, :a_cols]
            opB = B[:, :b_cols].T if tb else B[:, :b_cols]
            for alpha, beta in ((1.0, 0.0), (0.5, 1.0), (-2.0, 0.25)):
                want = C0.astype(np.float64).copy()
                want[:, :N] = alpha * (opA.astype(np.float64) @ opB.astype(np.float64)) + beta * want[:, :N]
                scale = max(1.0, np.abs(want).max())
                for allow, tol in ((None, 2e-3), (False, 2e-6)):
                    got = ref.backend_matmul("gpu", ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C0,
                                             ldc, allow_tf32=allow).reshape(M, ldc)
                    err = np.abs(got - want).max() / scale
                    assert err <= tol * np.sqrt(K), (shape, ta, tb, alpha, beta, allow, err)
                    # the padding columns of C are not part of the product: untouched
                    assert np.array_equal(got[:, N:], C0[:, N:])


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_network_runs_on_the_plugin(name, plugin_beside_host):
    case = CASES[name]
    args = (case["kind"], case["sizes"], case["batch"], case["T"], case["steps"])
    cpu = _run(*args, "cpu", case["hyper"], case.get("options"))
    gpu = _run(*args, "gpu", case["hyper"], case.get("options"))
    _compare(cpu, gpu, name)


CONV_ON_PLUGIN = ["conv_relu_small", "conv_ragged_geometry", "conv_adamw_center_projection"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", CONV_ON_PLUGIN)
def test_reference_conv_network_runs_on_the_plugin(name, plugin_beside_host):
    """SimpleConvPCNetwork of the reference on DEVICE_GPU: the plugin answers false to the fused
    convolution entries, so the host goes through Im2Col / Col2Im / RepackForBatchedGemm /
    MatMul[Batched] / AddBiasPerChannelNCHW of the plugin.  Compared with the same network on the
    reference's CPU backend: beliefs, weights, biases of every layer and a prediction.

    Not compared: the returned energy, the first layer's prediction and the error above it.  The
    reference's device path drops the clamped layer's cached prediction after recording its graph
    (src/networks/SimpleConvPCNetwork.cpp:147-161), so its closing energy evaluation uses the
    UPDATED weights there, while its CPU path keeps the prediction frozen for the whole step: the
    two differ by 30 % in energy on any backend, with identical parameters and beliefs."""
    from conv_common import CONV_CASES, run_conv_reference
    case = dict(CONV_CASES[name])
    cpu = run_conv_reference(case, "cpu")
    gpu = run_conv_reference(case, "gpu")
    worst, compared = 0.0, 0
    for key, want in cpu.items():
        kind = key.split(".")[-1]
        if key != "predict" and kind not in ("W", "b", "z"):
            continue
        got = gpu[key]
        err = float(np.max(np.abs(np.asarray(got, dtype=np.float64) - want) /
                           np.maximum(1.0, np.max(np.abs(want)))))
        worst = max(worst, err)
        compared += 1
        assert err <= 1e-2, (name, key, err)
    assert compared >= 2 * len(case["layers"])
    print(f"{name}: reference conv network on the plugin vs on its CPU backend, worst error {worst:.2e}")

"""GPU parity at the benchmark configurations themselves, against the COMPILED reference run
live on the host cores of the GPU box (oracle/_ref, the reference's own CPU code).

* the wide FullPCN workload at its shape: 3072-(1024x4)-10, GELU, softmax cross-entropy head,
  Adam for W and Psi, batch 4096, T = 20;
* the deep DKPPCN stack at its layer shape (width 512, batch 1024, T = 2, SGD) at depth 512 --
  or the largest of 256 / 128 the host's CPU finishes in about two minutes; the test prints
  which -- in the default fp32 mode (3xBF16 operand split) and with DPC_FP32_SCHEME=tf32x3;
* on request (DEEPITY_FULL_DEPTH_PARITY=1 and at least 128 GB of host memory) the energies of the
  full 2048-layer stack.

Compared: the energy of every step, every layer's z, e, W, b and Psi after the last step and a
prediction -- element by element for the deep stack (plus the parameter updates themselves,
relative to the largest update), as float64 sums and sums of squares per tensor for the wide
network.  Bounds: common.TOL (1e-4) for the SGD stack, common.ADAM_TOL (5e-4) for the Adam
network, common.DELTA_TOL on the updates.
The pattern is the reference's own CPU-vs-GPU differential test
(tests/tDirectKPBatchedGPUVerify.cpp:47-58,127-262), at a 100x tighter bound.
"""
import os
import sys
import time

import numpy as np
import pytest

from common import ADAM_TOL, DELTA_TOL, TOL, compare_outputs, initial_parameters, run_gpu

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

HYPER = dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0)


def _reference(case):
    from oracle import ref
    if not ref.available():
        pytest.skip("the compiled reference (oracle/_ref) is not present")
    from make_golden import run_reference
    t0 = time.perf_counter()
    out = run_reference(case)
    print(f"reference CPU run: {time.perf_counter() - t0:.1f} s "
          f"({ref.host_info()['omp_threads']} threads)")
    return out


def test_wide_fullpcn_at_its_benchmark_shape(built_library):
    case = dict(kind="full", sizes=[3072, 1024, 1024, 1024, 1024, 10], batch=4096, T=20, steps=2,
                stats_only=True, hyper=dict(act="gelu", **HYPER),
                options=dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM"))
    ref = _reference(case)
    worst = compare_outputs(ref, run_gpu(case, precision="fp32"), ADAM_TOL, "FullPCN at C4 shape")
    print(f"FullPCN 3072-(1024x4)-10 CE Adam B4096 T20: energies {ref['energies']}, "
          f"worst relative error {worst:.2e} (bound {ADAM_TOL})")


def _deep_case(depth, steps=2):
    return dict(kind="dkp", sizes=[512] + [512] * depth + [10], batch=1024, T=2, steps=steps,
                hyper=dict(act="tanh", **HYPER))


@pytest.fixture(scope="module")
def deep_reference():
    """The reference's outputs on the deepest stack this host's CPU handles in ~2 minutes."""
    from oracle import ref
    if not ref.available():
        pytest.skip("the compiled reference (oracle/_ref) is not present")
    from make_golden import run_reference
    t0 = time.perf_counter()
    run_reference(_deep_case(15, steps=1))
    per_layer = (time.perf_counter() - t0) / 16.0  # construction + one step
    depth = 512 if per_layer * 513 * 2 < 150 else 256 if per_layer * 257 * 2 < 150 else 128
    case = _deep_case(depth)
    t0 = time.perf_counter()
    out = run_reference(case)
    print(f"deep stack: depth {depth} ({per_layer * 1e3:.0f} ms per layer in the calibration run, "
          f"reference took {time.perf_counter() - t0:.1f} s)")
    return case, out, initial_parameters(case)


def test_deep_stack_default_fp32_scheme(built_library, deep_reference):
    case, ref, init = deep_reference
    worst = compare_outputs(ref, run_gpu(case, precision="fp32"), TOL, "deep stack 3xBF16",
                            init=init, delta_tol=DELTA_TOL)
    print(f"depth {len(case['sizes']) - 2}, 3xBF16 split: worst relative error {worst:.2e}")


def test_deep_stack_tf32x3_scheme(built_library, deep_reference, monkeypatch):
    case, ref, init = deep_reference
    monkeypatch.setenv("DPC_FP32_SCHEME", "tf32x3")
    worst = compare_outputs(ref, run_gpu(case, precision="fp32"), TOL, "deep stack 3xTF32",
                            init=init, delta_tol=DELTA_TOL)
    print(f"depth {len(case['sizes']) - 2}, 3xTF32 split: worst relative error {worst:.2e}")


def test_full_depth_energies(built_library):
    if os.environ.get("DEEPITY_FULL_DEPTH_PARITY") != "1":
        pytest.skip("set DEEPITY_FULL_DEPTH_PARITY=1 (the reference needs ~50 GB and minutes)")
    mem_gb = os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES") / 2 ** 30
    if mem_gb < 128:
        pytest.skip(f"host has {mem_gb:.0f} GB of memory; the 2048-layer reference needs 128")
    from oracle import ref as oref
    from common import build_gpu_net, make_case
    case = _deep_case(2048, steps=2)
    params, x, y = make_case("dkp", case["sizes"], 1024)
    net = oref.RefNet("dkp", case["sizes"], 1024, **case["hyper"])
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set(l, name, v)
    want = [net.train_step(x, y, 2) for _ in range(2)]
    del net
    gpu, _, _ = build_gpu_net(case, "fp32")
    got = [gpu.train_step(x, y, 2) for _ in range(2)]
    err = max(abs(a - b) / max(1.0, abs(a)) for a, b in zip(want, got))
    print(f"2048 layers: energies {want} vs {got}, relative difference {err:.2e}")
    assert err <= TOL

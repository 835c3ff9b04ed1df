"""GPU parity of the convolutional path: deepity_b200.SimpleConvolutionalPCN (implicit-GEMM
CUDA kernels behind the dpcn_conv_* C ABI) against the golden fixtures of the compiled
reference and the numpy oracle run live.  Bound: common.TOL per tensor (ADAM_TOL with an
Adam-type optimizer)."""
import os

import numpy as np
import pytest

from common import ADAM_TOL, TOL, compare_outputs
from conv_common import CONV_CASES, chain, run_conv_gpu, run_conv_oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def conv_tol(case):
    return ADAM_TOL if case.get("optimizer", "SGD") != "SGD" else TOL


@pytest.mark.parametrize("name", sorted(CONV_CASES))
def test_conv_gpu_matches_golden(name, built_library):
    case = CONV_CASES[name]
    ref = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    compare_outputs(ref, run_conv_gpu(case), conv_tol(case), name,
                    energy_tol=case.get("energy_tol"))


@pytest.mark.parametrize("name", ["conv_relu_small", "conv_zero_steps"])
def test_conv_gpu_without_graph(name, built_library):
    case = CONV_CASES[name]
    ref = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    compare_outputs(ref, run_conv_gpu(case, use_graph=False), conv_tol(case), name,
                    energy_tol=case.get("energy_tol"))


LIVE = {
    # channel counts and pixel counts that straddle the 64-wide tiles, batch not a power of two
    "conv_wide_channels": dict(layers=chain((5, 12, 12), [(70, 3, 3, 1, 1, 1, 1), (33, 5, 5, 2, 2, 2, 2),
                                                          (7, 6, 6, 1, 1, 0, 0)], "gelu"),
                               batch=6, T=3, steps=2, hyper=dict(lr=0.005, ir=0.1, lmbda=0.01)),
    "conv_batch_one_center": dict(layers=chain((3, 9, 9), [(4, 3, 3, 3, 3, 0, 0), (5, 3, 3, 1, 1, 0, 0)],
                                               "tanh"),
                                  batch=1, T=2, steps=3, center_weights=1,
                                  hyper=dict(lr=0.01, ir=0.2, lmbda=0.0)),
}


@pytest.mark.parametrize("name", sorted(LIVE))
def test_conv_gpu_matches_live_oracle(name, built_library):
    case = LIVE[name]
    compare_outputs(run_conv_oracle(case), run_conv_gpu(case), conv_tol(case), name,
                    energy_tol=case.get("energy_tol"))


def test_conv_energy_decreases(built_library):
    # the sanity property of tests/tSimpleConvPCNetworkTrainStepSanity.cpp in the reference
    case = dict(CONV_CASES["conv_tanh_sanity_shape"], steps=20)
    e = run_conv_gpu(case)["energies"]
    assert np.all(np.isfinite(e)) and e[-1] < e[0]

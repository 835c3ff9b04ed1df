"""Pins the numpy restatement of the convolutional path (oracle/conv_oracle.py) to the
reference: every golden fixture (outputs of the compiled reference's SimpleConvPCNetwork), the
compiled reference run live when it is present, and the finite-difference property the
reference's own test checks (tests/tSimpleConvPCLayerStateVerify.cpp: with ir = 1 a state
update moves an unclamped middle layer by -dE/dz)."""
import os

import numpy as np
import pytest

from common import ADAM_TOL, TOL, compare_outputs
from conv_common import CONV_CASES, chain, make_conv_case, run_conv_oracle, run_conv_reference

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def conv_tol(case):
    return ADAM_TOL if case.get("optimizer", "SGD") != "SGD" else TOL


@pytest.mark.parametrize("name", sorted(CONV_CASES))
def test_conv_oracle_matches_golden(name):
    case = CONV_CASES[name]
    ref = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    compare_outputs(ref, run_conv_oracle(case), conv_tol(case), name,
                    energy_tol=case.get("energy_tol"))


@pytest.mark.parametrize("name", ["conv_relu_small", "conv_zero_steps", "conv_ragged_geometry"])
def test_conv_oracle_matches_compiled_reference_live(name):
    from oracle import ref as oref
    if not oref.available():
        pytest.skip("compiled reference not present")
    case = CONV_CASES[name]
    compare_outputs(run_conv_reference(case), run_conv_oracle(case), conv_tol(case), name,
                    energy_tol=case.get("energy_tol"))


def test_state_update_is_minus_energy_gradient():
    from oracle.conv_oracle import ConvOracle
    layers = chain((1, 6, 6), [(2, 3, 3, 1, 1, 0, 0), (3, 2, 2, 1, 1, 0, 0)], "tanh")
    case = dict(layers=layers, batch=1, seed=4)
    params, x, y = make_conv_case(case)
    net = ConvOracle(layers, 1, lr=0.0, ir=1.0, lmbda=0.0)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set(l, nm, v)
    net.reset()
    net.clamp(0, x)
    net.clamp(2, y)
    mid = net.layers[1]
    mid.z[...] = np.random.default_rng(1).normal(0, 0.5, mid.z.shape).astype(np.float32)

    def energy():
        return float(sum(net.calculate_state(i, True) for i in range(3)))
    energy()
    before = mid.z.copy()
    net.update_state(1)
    analytic = -(mid.z - before)
    mid.z[...] = before
    eps = 3e-3
    for idx in [(0, 0, 1, 2), (0, 1, 3, 0), (0, 1, 2, 2)]:
        mid.z[idx] = before[idx] + eps
        ep = energy()
        mid.z[idx] = before[idx] - eps
        em = energy()
        mid.z[idx] = before[idx]
        numeric = (ep - em) / (2 * eps)
        assert abs(numeric - analytic[idx]) <= 1e-2 * (abs(numeric) + 1e-6) + 1e-3, (idx, numeric,
                                                                                   analytic[idx])

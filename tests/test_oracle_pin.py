"""CPU tests: the numpy oracle is pinned against the compiled reference's outputs.

* every golden fixture under tests/golden (outputs of the reference's own CPU code, made by
  tests/golden/make_golden.py);
* the compiled reference itself, live, when oracle/_ref is present (fresh seeds);
* the known-answer / independent-reference checks the reference's own tests hold for the
  primitives on this path (tests/tAddBiasBroadcastVerify.cpp:41-46,
  tests/tCrossEntropyVerify.cpp:14-45, tests/tFullPCMomentumVerify.cpp:100-134 there).
"""
import json
import os

import numpy as np
import pytest

from common import ADAM_TOL, TOL, compare_outputs, make_case, make_oracle, rel_err, run_oracle
from oracle import pc_oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = json.load(open(os.path.join(GOLDEN, "cases.json")))


def case_tol(case):
    o = case.get("options", {})
    adam = o.get("optimizer", "SGD") != "SGD" or o.get("psi_optimizer", "SGD") != "SGD"
    return ADAM_TOL if adam else TOL


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_golden(name):
    case = CASES[name]
    ref = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    got = run_oracle(case)
    compare_outputs(ref, got, case_tol(case), name)


def test_oracle_matches_compiled_reference_live():
    from oracle import ref as oref
    if not oref.available():
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    kind, sizes, B, T = "dkp", [24, 40, 40, 40, 10], 20, 2
    params, x, y = make_case(kind, sizes, B, seed=7)
    hyper = dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")
    net = oref.RefNet(kind, sizes, B, **hyper)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set(l, nm, v)
    orc = make_oracle(kind, sizes, B, params, **hyper)
    for _ in range(3):
        er, eo = net.train_step(x, y, T), orc.train_step(x, y, T)
        assert abs(er - eo) <= TOL * max(1.0, abs(er))
    for l in range(net.num_layers):
        for nm in ("z", "e", "W", "b", "Psi"):
            a = net.get(l, nm)
            if a.size:
                assert rel_err(a, orc.get(l, nm)) <= TOL, (l, nm)


def test_add_bias_broadcast_known_answer():
    # tests/tAddBiasBroadcastVerify.cpp:41-46 of the reference
    buf = np.array([1, 2, 3, 4, 10, 20, 30, 40, 100, 200, 300, 400], np.float32).reshape(3, 4)
    bias = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    expected = np.array([1.1, 2.2, 3.3, 4.4, 10.1, 20.2, 30.3, 40.4, 100.1, 200.2, 300.3, 400.4],
                        np.float32)
    L = pc_oracle._Layer(4, 4, 4, 3, 0, 0, 0, 0, "linear")
    L.W[...] = np.eye(4, dtype=np.float32)
    L.b[...] = bias
    L.z[...] = buf
    o = pc_oracle.PCOracle("dkp", [4, 4], 3)
    o.layers[0] = L
    o.compute_mu(L)
    assert np.abs(L.mu.ravel() - expected).max() <= 1e-4


def test_softmax_ce_against_independent_reference():
    # the double-precision restatement of tests/tCrossEntropyVerify.cpp:14-45
    rng = np.random.default_rng(3)
    mu = rng.normal(0, 3, (7, 10)).astype(np.float32)
    z = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 7)]
    e, energy = pc_oracle.softmax_ce(z, mu)
    m64 = mu.astype(np.float64)
    p = np.exp(m64 - m64.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    assert np.abs(e - (z - p)).max() < 1e-4
    assert abs(energy - float(-(z * np.log(p + 1e-8)).sum())) < 1e-3


def test_momentum_recurrence():
    # v = beta v + (1-beta)(fe.(aW) - e); z += ir v   (tests/tFullPCMomentumVerify.cpp:100-134)
    beta, ir = np.float32(0.75), np.float32(0.1)
    o = pc_oracle.PCOracle("full", [6, 5, 4], 3, ir=float(ir), momentum=float(beta))
    rng = np.random.default_rng(5)
    L, up = o.layers[1], o.layers[2]
    L.W[...] = rng.normal(size=L.W.shape)
    L.z[...] = rng.normal(size=L.z.shape)
    L.e[...] = rng.normal(size=L.e.shape)
    L.preact[...] = rng.normal(size=L.preact.shape)
    up.e[...] = rng.normal(size=up.e.shape)
    v = np.zeros_like(L.z)
    z = L.z.copy()
    for _ in range(3):
        upd = (up.e * pc_oracle.dact("tanh", L.preact)) @ L.W - L.e
        v = beta * v + (np.float32(1) - beta) * upd
        z = z + ir * v
        o.update_state(1)
    assert np.abs(L.z - z).max() < 1e-4


def test_adam_first_step_is_lr_sized():
    p = np.array([1.0, -2.0, 0.5], np.float32)
    g = np.array([0.3, -0.1, 2.0], np.float32)
    m, v = np.zeros(3, np.float32), np.zeros(3, np.float32)
    pc_oracle.adam_step(p, g, m, v, 1, 1e-2)
    assert np.allclose(p, np.array([1.0, -2.0, 0.5]) - 1e-2 * np.sign(g), atol=1e-6)

"""Checkpoint surface on the GPU: the reference's tensor names, shapes and optimizer step
counters (Layer::GetStateDict / GetOptimizerStateDict / GetOptimizerCounters,
include/deepity/layers/Layer.h:100-134, src/layers/DirectKPPCLayer.cpp:219-241) read from and
written to the device layout through the C ABI."""
import numpy as np
import pytest

from common import build_gpu_net

pytestmark = pytest.mark.gpu

CASE = dict(kind="dkp", sizes=[20, 48, 48, 10], batch=16, T=2, steps=3,
            hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.01, act="gelu"),
            options=dict(optimizer="ADAMW", psi_optimizer="ADAM"))


def test_names_and_shapes_follow_the_reference(built_library):
    net, x, y = build_gpu_net(CASE)
    net.train_step(x, y, 2)
    sd, osd = net.state_dict(), net.optimizer_state_dict()
    assert sorted(sd) == sorted(f"layers.{l}.{n}" for l in range(3) for n in ("weight", "bias", "psi"))
    assert sd["layers.0.weight"].shape == (48, 20) and sd["layers.0.bias"].shape == (48,)
    assert sd["layers.1.psi"].shape == (48, 10) and sd["layers.2.weight"].shape == (10, 48)
    for l in range(3):
        for n in ("weight.m", "weight.v", "bias.m", "bias.v", "psi.m", "psi.v"):
            assert f"optimizer.layers.{l}.{n}" in osd
        assert osd[f"optimizer.layers.{l}.step"].tolist() == [1]
        assert osd[f"optimizer.layers.{l}.psi_step"].tolist() == [1]
        assert osd[f"optimizer.layers.{l}.psi.m"].shape == sd[f"layers.{l}.psi"].shape


def test_sgd_network_has_no_optimizer_state(built_library):
    case = dict(CASE, options={})
    net, x, y = build_gpu_net(case)
    net.train_step(x, y, 2)
    assert net.optimizer_state_dict() == {}


def test_resumed_adam_run_matches_bit_for_bit(built_library):
    """Two steps, checkpoint, restore into a FRESH network, third step: every tensor equals
    the uninterrupted run's (the Adam bias correction depends on the restored counters)."""
    a, x, y = build_gpu_net(CASE)
    for _ in range(2):
        a.train_step(x, y, 2)
    ckpt = {**a.state_dict(), **a.optimizer_state_dict()}
    b, _, _ = build_gpu_net(CASE)
    rng = np.random.default_rng(7)
    for l in range(3):  # make sure the restore does the work, not the common seed
        b.set_tensor(l, "W", rng.normal(size=b.get_tensor(l, "W").shape).astype(np.float32))
    b.load_state_dict(ckpt)
    ea, eb = a.train_step(x, y, 2), b.train_step(x, y, 2)
    assert ea == eb
    for k, v in a.state_dict().items():
        assert np.array_equal(v, b.state_dict()[k]), k
    for k, v in a.optimizer_state_dict().items():
        assert np.array_equal(v, b.optimizer_state_dict()[k]), k
    assert b.optimizer_state_dict()["optimizer.layers.0.step"].tolist() == [3]


def test_strict_load_reports_missing_tensors(built_library):
    net, x, y = build_gpu_net(CASE)
    sd = net.state_dict()
    del sd["layers.1.bias"]
    with pytest.raises(KeyError):
        net.load_state_dict(sd)
    net.load_state_dict(sd, strict=False)

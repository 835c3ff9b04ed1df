"""CPU tests (gloo, world_size 2 and 3) of the layer-sharding schedule.

The schedule of deepity_b200/sharded.py — which boundary tensor goes where in which phase —
runs here over an engine backed by the numpy oracle, one block of layers per CPU rank, and
must reproduce the single-process oracle: energies of every step and every tensor.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from common import TOL, make_case, make_oracle, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleEngine:
    """The engine interface of deepity_b200.sharded.GpuEngine over oracle.pc_oracle."""

    def __init__(self, sizes, batch, hyper, act, ghost_top, terminal_size):
        from oracle.pc_oracle import PCOracle
        self.o = PCOracle("dkp", sizes, batch, act=act, terminal_size=terminal_size, **hyper)
        self.n = len(sizes)
        self.ghost_top = ghost_top
        self.energy = 0.0
        if ghost_top:
            g = self.o.layers[-1]
            g.Psi = np.zeros((g.s, terminal_size), np.float32)
            self.eT = np.zeros((batch, terminal_size), np.float32)
            self.o.e_terminal = self.eT

    def tensor(self, layer, name):
        a = self.eT if name == "eT" else getattr(self.o.layers[layer], name)
        return torch.from_numpy(a.reshape(-1))

    def terminal_error_tensor(self):
        return self.tensor(self.n - 1, "eT" if self.ghost_top else "e")

    def set_param(self, layer, name, value):
        self.o.set(layer, name, value)

    def get(self, layer, name):
        return np.array(getattr(self.o.layers[layer], name)).ravel()

    def reset(self):
        self.o.reset()
        for L in self.o.layers:
            L.clamped = False

    def wrote_belief(self, layer):
        pass

    def mark_clamped(self, layer):
        self.o.layers[layer].clamped = True
        self.o.layers[layer].cache_valid = False

    def project_forward(self, skip_last_copy):
        for i in range(self.n - 1):
            self.o.compute_mu(self.o.layers[i])
            if not (skip_last_copy and i + 2 == self.n):
                self.o.layers[i + 1].z[...] = self.o.layers[i].mu

    def terminal_error(self):
        self.o.calculate_state(self.n - 1, False)

    def dfa(self):
        for i in range(self.n - 1):
            self.o.dfa(i)

    def forward_state(self, first_cached, flags):
        for i in range(self.n - 1):
            self.o.compute_mu(self.o.layers[i])
            if flags & 2:
                up = self.o.layers[i + 1]
                up.e[...] = up.z - self.o.layers[i].mu
                if flags & 4:
                    self.energy += float(np.float32(0.5) * (up.e * up.e).sum(dtype=np.float32))

    def update_state(self, first, count):
        for i in range(first, first + count):
            self.o.update_state(i)

    def update_weights(self):
        for i in range(self.n - 1):
            self.o.update_weights(i)

    def energy_reset(self):
        self.energy = 0.0

    def energy_read(self):
        return self.energy

    def sync(self):
        pass

    def comm_stream(self):
        import contextlib
        return contextlib.nullcontext()


CASE = dict(kind="dkp", sizes=[12, 20, 20, 20, 20, 20, 6], batch=8, T=2, steps=3,
            hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0), act="tanh")


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepity_b200.sharded import ShardedDKPPCN
    params, x, y = make_case("dkp", CASE["sizes"], CASE["batch"], seed=3)
    net = ShardedDKPPCN(CASE["sizes"], CASE["batch"], CASE["hyper"], act=CASE["act"],
                        engine_factory=OracleEngine)
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_param(l, nm, v)
    energies = [net.train_step(x, y, CASE["T"]) for _ in range(CASE["steps"])]
    res = {"energies": energies}
    for l in range(net.begin, net.end):
        for nm in ("z", "e", "W", "b", "Psi"):
            res[f"{l}.{nm}"] = net.get_local(l, nm)
    if net.is_last:
        res[f"{net.end}.z"] = net.get_local(net.end, "z")
        res[f"{net.end}.e"] = net.get_local(net.end, "e")
    # checkpoint surface: the whole network's tensors by global name on rank 0, and back
    gathered = net.gather_state_dict(dst=0)
    if rank == 0:
        res["state_dict"] = {k: np.array(v) for k, v in gathered.items()}
    else:
        assert gathered is None
    state = [gathered]
    dist.broadcast_object_list(state, src=0)
    net.load_state_dict(state[0])
    for l in range(net.begin, net.end):
        assert np.array_equal(np.asarray(net.get_local(l, "W")).ravel(), res[f"{l}.W"].ravel())
    out[rank] = res
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_schedule_matches_single_process_oracle(world):
    from deepity_b200.sharded import partition_layers
    assert partition_layers(6, 3) == [(0, 2), (2, 4), (4, 6)]
    assert partition_layers(7, 3) == [(0, 3), (3, 5), (5, 7)]
    with pytest.raises(ValueError):
        partition_layers(2, 3)

    params, x, y = make_case("dkp", CASE["sizes"], CASE["batch"], seed=3)
    ref = make_oracle("dkp", CASE["sizes"], CASE["batch"], params, act=CASE["act"], **CASE["hyper"])
    ref_e = [ref.train_step(x, y, CASE["T"]) for _ in range(CASE["steps"])]

    mgr = mp.Manager()
    out = mgr.dict()
    port = 29500 + (os.getpid() % 1000) + world
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        for a, b in zip(out[r]["energies"], ref_e):
            assert abs(a - b) <= TOL * max(1.0, abs(b)), (r, a, b)
    sd = out[0]["state_dict"]
    n_w = len(CASE["sizes"]) - 1
    assert sorted(sd) == sorted(f"layers.{l}.{n}" for l in range(n_w) for n in ("weight", "bias", "psi"))
    for l in range(n_w):
        assert sd[f"layers.{l}.weight"].shape == (CASE["sizes"][l + 1], CASE["sizes"][l])
        assert rel_err(ref.get(l, "W"), sd[f"layers.{l}.weight"]) <= TOL
        assert rel_err(ref.get(l, "Psi"), sd[f"layers.{l}.psi"]) <= TOL
    seen = set()
    for r in range(world):
        for key, val in out[r].items():
            if key in ("energies", "state_dict"):
                continue
            l, nm = key.split(".")
            assert rel_err(ref.get(int(l), nm), val) <= TOL, key
            seen.add(key)
    n_weight = len(CASE["sizes"]) - 1
    assert all(f"{l}.W" in seen for l in range(n_weight))

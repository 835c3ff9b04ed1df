"""CPU tests (gloo, world_size 2 and 4) of batch sharding.

deepity_b200.sharded.BatchSharded runs here over the numpy oracle, one slice of batch rows
per CPU rank with the gradient sums all-reduced, and must reproduce the single-process oracle
on the whole batch: the energy of every step and W, b, Psi on every rank.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from common import ADAM_TOL, TOL, _oracle_kwargs, make_case, make_oracle, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleShard:
    """oracle.pc_oracle.PCOracle behind the set_gradient_sync / train_step pair."""

    def __init__(self, case, local_batch, params):
        self.case = case
        self.o = make_oracle(case["kind"], case["sizes"], local_batch, params,
                             **_oracle_kwargs(case))

    def set_gradient_sync(self, reduce_fn, global_batch):
        def hook(phase, layer, arrays):
            live = [a for a in arrays if a is not None]
            flat = torch.from_numpy(np.concatenate([np.asarray(a, np.float32).ravel()
                                                    for a in live]))
            reduce_fn(flat)
            out, pos = [], 0
            for a in arrays:
                if a is None:
                    out.append(None)
                    continue
                out.append(flat[pos:pos + a.size].numpy().reshape(a.shape).copy())
                pos += a.size
            return out
        self.o.grad_sync = hook
        self.o.global_B = global_batch

    def train_step(self, x, y, T):
        return self.o.train_step(x, y, T)


CASES = {
    "full_ce_adam": dict(kind="full", sizes=[12, 16, 16, 5], batch=8, T=3, steps=3,
                         hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="gelu"),
                         options=dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM")),
    "full_ipc_sgd": dict(kind="full", sizes=[12, 16, 16, 5], batch=8, T=3, steps=2,
                         hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="tanh"),
                         options=dict(ipc=1)),
    "dkp_sgd": dict(kind="dkp", sizes=[12, 16, 16, 5], batch=8, T=2, steps=3,
                    hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "simple_sgd": dict(kind="simple", sizes=[12, 16, 5], batch=8, T=4, steps=2,
                       hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="sigmoid")),
}


def _worker(rank, world, port, name, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepity_b200.sharded import BatchSharded
    case = CASES[name]
    params, x, y = make_case(case["kind"], case["sizes"], case["batch"], seed=5)
    net = BatchSharded(lambda b: OracleShard(case, b, params), case["batch"])
    energies = [net.train_step(x, y, case["T"]) for _ in range(case["steps"])]
    res = {"energies": energies}
    o = net.net.o
    for l in range(len(case["sizes"]) - 1):
        for nm in ("W", "b") + (() if case["kind"] == "simple" else ("Psi",)):
            res[f"{l}.{nm}"] = np.array(o.get(l, nm)).ravel()
    out[rank] = res
    dist.destroy_process_group()


@pytest.mark.parametrize("world,name", [(2, "full_ce_adam"), (2, "full_ipc_sgd"), (2, "dkp_sgd"),
                                        (2, "simple_sgd"), (4, "full_ce_adam")])
def test_batch_sharded_matches_single_process_oracle(world, name):
    case = CASES[name]
    params, x, y = make_case(case["kind"], case["sizes"], case["batch"], seed=5)
    ref = make_oracle(case["kind"], case["sizes"], case["batch"], params, **_oracle_kwargs(case))
    ref_e = [ref.train_step(x, y, case["T"]) for _ in range(case["steps"])]
    tol = ADAM_TOL if case.get("options", {}).get("optimizer", "SGD") != "SGD" else TOL

    mgr = mp.Manager()
    out = mgr.dict()
    port = 29700 + (os.getpid() % 1000) + world
    mp.spawn(_worker, args=(world, port, name, out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        for a, b in zip(out[r]["energies"], ref_e):
            assert abs(a - b) <= tol * max(1.0, abs(b)), (r, a, b)
        for key, val in out[r].items():
            if key == "energies":
                continue
            l, nm = key.split(".")
            assert rel_err(ref.get(int(l), nm), val) <= tol, (r, key)


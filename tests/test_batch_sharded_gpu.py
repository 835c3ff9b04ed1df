"""Batch sharding on real GPUs (needs two): FullPCN with a softmax head and Adam, the global
batch split over two ranks with NCCL all-reduces of the staged gradients, against the
single-process oracle on the whole batch."""
import os
import sys

import numpy as np
import pytest

from common import ADAM_TOL, build_gpu_net, make_case, rel_err, run_oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASE = dict(kind="full", sizes=[48, 64, 64, 10], batch=32, T=3, steps=3,
            hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="gelu"),
            options=dict(cross_entropy=1, optimizer="ADAM", psi_optimizer="ADAM"))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    from deepity_b200.sharded import BatchSharded
    _, x, y = make_case(CASE["kind"], CASE["sizes"], CASE["batch"], seed=CASE.get("seed", 0))

    def build(local_batch):
        net, _, _ = build_gpu_net(dict(CASE, batch=local_batch), device=f"cuda:{rank}")
        return net
    net = BatchSharded(build, CASE["batch"])
    energies = [net.train_step(x, y, CASE["T"]) for _ in range(CASE["steps"])]
    res = {"energies": energies}
    for l in range(len(CASE["sizes"]) - 1):
        for nm in ("W", "b", "Psi"):
            res[f"t.{l}.{nm}"] = net.net.get_tensor(l, nm)
    out[rank] = res
    dist.destroy_process_group()


def test_two_gpu_batch_sharded_fullpcn(built_library):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ref = run_oracle(CASE)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, 29900 + os.getpid() % 500, out), nprocs=2, join=True)
    for r in range(2):
        for a, b in zip(out[r]["energies"], ref["energies"]):
            assert abs(a - b) <= ADAM_TOL * max(1.0, abs(b)), (r, a, b)
        for key, val in out[r].items():
            if key != "energies":
                assert rel_err(ref[key], val) <= ADAM_TOL, (r, key)

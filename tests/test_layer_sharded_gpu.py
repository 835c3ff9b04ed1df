"""Layer sharding on real GPUs (needs two): a DKPPCN split over two ranks with NCCL
send/recv of the boundary tensors, against the single-process oracle on the whole network."""
import os
import sys

import pytest

from common import TOL, make_case, make_oracle, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SIZES = [64] + [256] * 9 + [10]
BATCH, T, STEPS = 128, 2, 3
HYPER = dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    from deepity_b200.sharded import ShardedDKPPCN
    params, x, y = make_case("dkp", SIZES, BATCH, seed=5)
    net = ShardedDKPPCN(SIZES, BATCH, HYPER, act="tanh", precision="fp32")
    for l, p in enumerate(params):
        for nm, v in p.items():
            net.set_param(l, nm, v)
    res = {"energies": [net.train_step(x, y, T) for _ in range(STEPS)]}
    for l in range(net.begin, net.end):
        for nm in ("z", "e", "W", "b", "Psi"):
            res[f"{l}.{nm}"] = net.get_local(l, nm)
    out[rank] = res
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_layer_sharded_dkppcn(built_library):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    params, x, y = make_case("dkp", SIZES, BATCH, seed=5)
    ref = make_oracle("dkp", SIZES, BATCH, params, act="tanh", **HYPER)
    ref_e = [ref.train_step(x, y, T) for _ in range(STEPS)]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, 29950 + os.getpid() % 500, out), nprocs=2, join=True)
    assert len(out) == 2
    for r in range(2):
        for a, b in zip(out[r]["energies"], ref_e):
            assert abs(a - b) <= TOL * max(1.0, abs(b)), (r, a, b)
        for key, val in out[r].items():
            if key != "energies":
                l, nm = key.split(".")
                assert rel_err(ref.get(int(l), nm), val) <= TOL, (r, key)

"""Failure detection on the device without faulting it: every wait inside the tensor-core
kernels is bounded, and a wait that runs out is reported to the host as DPC_ERR_TIMEOUT while
the CUDA context stays usable.

The failure is made on the host side: the wait limit is set to 2 ms and the forward sweep is
told to wait for one publication more per row block than its producers will ever make (a flag
that nothing sets).  The kernel's waiting roles give up after the limit, raise the status flag,
let their copies in flight land, free their tensor memory and return; the step's remaining
kernels run on whatever is in memory; the energy read at the end of the step reports the
time-out.  With the limit and the target restored and the parameters reloaded, the same step
then gives the same energy as before."""
import ctypes

import numpy as np
import pytest

from common import build_gpu_net, make_case

pytestmark = pytest.mark.gpu

CASE = dict(kind="dkp", sizes=[512] * 7 + [10], batch=1024, T=2, steps=1,
            hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh"))


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(built_library):
    import deepity_b200 as dp
    from deepity_b200 import _lib
    lib = _lib.load()
    net, x, y = build_gpu_net(CASE, "fp32", use_graph=False)
    plan = lib.dpcn_plan(net._h)
    first, count = ctypes.c_int(), ctypes.c_int()
    lib.dpc_plan_tensor_run(plan, ctypes.byref(first), ctypes.byref(count))
    assert count.value >= 2, "the case must use the persistent forward sweep"
    good = net.train_step(x, y, CASE["T"])
    assert np.isfinite(good)

    _lib.check(lib.dpc_plan_set_wait_limit(plan, 2.0, 1))
    with pytest.raises(dp.DeepityError) as err:
        net.train_step(x, y, CASE["T"])
    assert err.value.status == -5  # DPC_ERR_TIMEOUT
    assert "gave up waiting" in str(err.value)

    # back to normal: default limit, real target, the parameters the first step started from
    _lib.check(lib.dpc_plan_set_wait_limit(plan, 0.0, 0))
    params, _, _ = make_case(CASE["kind"], CASE["sizes"], CASE["batch"])
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set_tensor(l, name, v)
    again = net.train_step(x, y, CASE["T"])
    assert abs(again - good) <= 1e-6 * max(1.0, abs(good)), (good, again)

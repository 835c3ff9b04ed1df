"""The epoch loop: with the data set resident on the device (mini-batches gathered there through
dpc_gather_rows) it visits the same batches as the host-sliced loop of the reference
(deepity/utils.py:19-143) and ends with bit-identical parameters."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _net():
    import deepity_b200 as dp
    net = dp.DKPPCN(dp.Linear(20, 32), dp.TanH(), dp.Linear(32, 32), dp.TanH(), dp.Linear(32, 5),
                    batch_size=16)
    net.configure(learning_rate=0.01, inference_rate=0.1, feedback_rate=0.01, lmbda=0.0,
                  optimizer="SGD", psi_optimizer="SGD", seed=3)
    return net


def test_device_resident_fit_matches_host_sliced_fit(built_library):
    rng = np.random.default_rng(5)
    X = rng.standard_normal((96, 20)).astype(np.float32)
    Y = np.eye(5, dtype=np.float32)[rng.integers(0, 5, 96)]
    results = []
    for resident in (False, True):
        net = _net()
        np.random.seed(11)
        net.fit(X, Y, epochs=3, inference_steps=2, decay_rate=0.9, device_resident=resident)
        results.append([np.array(net.get_tensor(l, name)) for l in range(3)
                        for name in ("W", "b", "Psi")])
    for host, dev in zip(*results):
        assert np.array_equal(host, dev)


def test_gather_rows_ragged_width(built_library):
    import ctypes
    import torch
    from deepity_b200 import _lib
    lib = _lib.load()
    net = _net()
    ctx = lib.dpcn_context(net._h)
    stream = torch.cuda.ExternalStream(lib.dpc_stream(ctx))
    with torch.cuda.stream(stream):
        src = torch.arange(50 * 7, dtype=torch.float32, device="cuda").reshape(50, 7)
        idx = torch.tensor([4, 49, 0, 17, 17, 3], dtype=torch.int64, device="cuda")
        dst = torch.zeros((4, 7), dtype=torch.float32, device="cuda")
        _lib.check(lib.dpc_gather_rows(ctx, ctypes.c_void_p(src.data_ptr()),
                                       ctypes.c_void_p(idx.data_ptr()), 1, 4, 7,
                                       ctypes.c_void_p(dst.data_ptr())))
        stream.synchronize()
    assert torch.equal(dst.cpu(), src.cpu()[[49, 0, 17, 17]])

"""GPU test of dpc_error_energy_static, the entry point that allocates nothing.

It exists for callers that cannot obtain device memory at call time — a service whose GPU
memory belongs to a framework pool, a loop that may not allocate once it runs, code between
graph captures — so its reduction scratch is a static device array.  The test calls it through
the C ABI twice in a row on device buffers the test owns and checks the error tensor (bit for
bit) and the energy (1e-6 relative: only the summation order differs) against the ordinary
entry points dpc_error + dpc_energy_read on the same data; the second call also proves that
the shared scratch is left clean by the first.  The file sorts last so that a failure here
cannot hide any other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_entry_matches_plan_entry_twice(built_library):
    import json
    import os
    from common import build_gpu_net
    from deepity_b200 import _lib

    lib = _lib.load()
    cases = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "cases.json")))
    case = cases["dkp_tanh_small"]
    net, x, y = build_gpu_net(case)
    net.train_step(x, y, case["T"])  # leaves valid z / mu behind
    ctx, plan = lib.dpcn_context(net._h), lib.dpcn_plan(net._h)
    layer = 2
    B, s = case["batch"], case["sizes"][layer]
    n = B * s
    rng = np.random.default_rng(11)

    def ptr(l, name):
        p, stride = ctypes.c_void_p(), ctypes.c_int64()
        _lib.check(lib.dpcn_tensor_ptr(net._h, l, name.encode(), ctypes.byref(p),
                                       ctypes.byref(stride)))
        return p

    e_out, en_out = ctypes.c_void_p(), ctypes.c_void_p()
    _lib.check(lib.dpc_alloc(ctx, n * 4, ctypes.byref(e_out)))
    _lib.check(lib.dpc_alloc(ctx, 4, ctypes.byref(en_out)))
    try:
        for call in range(2):
            z = rng.normal(size=(B, s)).astype(np.float32)
            net.set_tensor(layer, "z", z)
            # ordinary path: error of `layer` against the prediction below, energy via the plan
            _lib.check(lib.dpc_energy_reset(plan))
            _lib.check(lib.dpc_error(plan, layer, 1))
            ref_energy = ctypes.c_double()
            _lib.check(lib.dpc_energy_read(plan, ctypes.byref(ref_energy)))
            ref_e = net.get_tensor(layer, "e")
            # static path on the same z and mu, into buffers of our own
            _lib.check(lib.dpc_error_energy_static(lib.dpc_stream(ctx), ptr(layer, "z"),
                                                   ptr(layer - 1, "mu"), e_out, n, en_out))
            got_e = np.empty(n, np.float32)
            got_energy = np.empty(1, np.float32)
            _lib.check(lib.dpc_copy_d2h_sync(ctx, got_e.ctypes.data_as(ctypes.c_void_p), e_out, n * 4))
            _lib.check(lib.dpc_copy_d2h_sync(ctx, got_energy.ctypes.data_as(ctypes.c_void_p),
                                             en_out, 4))
            assert np.array_equal(got_e, ref_e), f"call {call}: error tensor differs"
            assert abs(float(got_energy[0]) - ref_energy.value) <= 1e-6 * max(1.0, ref_energy.value), \
                (call, float(got_energy[0]), ref_energy.value)
            mu = net.get_tensor(layer - 1, "mu")
            expect = 0.5 * float(((z.ravel().astype(np.float64) - mu) ** 2).sum())
            assert abs(float(got_energy[0]) - expect) <= 1e-5 * max(1.0, expect)
    finally:
        lib.dpc_free(ctx, e_out)
        lib.dpc_free(ctx, en_out)


def test_static_entry_rejects_oversize_and_null(built_library):
    from deepity_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    assert lib.dpc_error_energy_static(None, one, one, one, (1 << 26) + 1, one) == -6
    assert b"fixed maximum" in lib.dpc_last_error()
    assert lib.dpc_error_energy_static(None, None, one, one, 16, one) == -1

"""CPU tests of the boundary: the shared library loads, exports every symbol the header
declares with the signature table the Python loader uses, and fails loudly (no fallback)
when there is no CUDA device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "deepity_b200.h")).read()
    return sorted(set(re.findall(r"DPC_API\s+[\w\s\*]+?\b(dpcn?_\w+)\s*\(", text)))


def test_header_declares_a_sane_surface():
    syms = header_symbols()
    assert len(syms) >= 50
    for must in ("dpc_create", "dpc_forward", "dpc_update_state", "dpc_update_weights",
                 "dpc_direct_feedback", "dpcn_train_step", "dpcn_predict"):
        assert must in syms


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    missing = [s for s in header_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_loader_table_matches_header(built_library):
    from deepity_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_symbols()
    _lib.load()


def test_no_device_is_a_loud_error(built_library):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from deepity_b200 import _lib
    lib = _lib.load()
    h = ctypes.c_void_p()
    rc = lib.dpc_create(0, ctypes.byref(h))
    assert rc == -2  # DPC_ERR_NO_DEVICE
    assert b"no CPU fallback" in lib.dpc_last_error()
    import deepity_b200 as dp
    with pytest.raises(dp.DeepityError):
        dp.DKPPCN(dp.Linear(4, 4), batch_size=2)


def test_bad_arguments_are_rejected(built_library):
    from deepity_b200 import _lib
    lib = _lib.load()
    assert lib.dpc_create(0, None) == -1
    assert lib.dpcn_create(7, 8, 0, None) == -1
    assert lib.dpc_forward(None, 0, 1, 0) == -1
    assert lib.dpc_energy_read(None, None) == -1
    import deepity_b200 as dp
    with pytest.raises(ValueError):
        dp.DKPPCN(dp.Linear(4, 5), dp.Linear(6, 3), batch_size=2)
    with pytest.raises(TypeError):
        dp.DKPPCN(dp.TanH(), batch_size=2)

"""ctypes loader for libdeepity_b200.so (the C ABI declared in include/deepity_b200.h).

There is no Python or CPU fallback: if the shared library is missing the import fails with
instructions to build it, and every compute call fails with a clear error when no CUDA
device is present.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libdeepity_b200.so")

c_f32p = ctypes.POINTER(ctypes.c_float)
_i, _f, _vp, _cp, _i64 = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int64

# name -> (restype, argtypes); every symbol include/deepity_b200.h declares.
SIGNATURES = {
    "dpc_last_error": (_cp, []),
    "dpc_version": (_cp, []),
    "dpc_create": (_i, [_i, ctypes.POINTER(_vp)]),
    "dpc_destroy": (_i, [_vp]),
    "dpc_set_precision": (_i, [_vp, _i]),
    "dpc_get_precision": (_i, [_vp]),
    "dpc_stream": (_vp, [_vp]),
    "dpc_launch_count": (_i64, [_vp]),
    "dpc_alloc": (_i, [_vp, ctypes.c_size_t, ctypes.POINTER(_vp)]),
    "dpc_free": (_i, [_vp, _vp]),
    "dpc_zero": (_i, [_vp, _vp, ctypes.c_size_t]),
    "dpc_copy_d2d": (_i, [_vp, _vp, _vp, ctypes.c_size_t]),
    "dpc_copy_h2d": (_i, [_vp, _vp, _vp, ctypes.c_size_t]),
    "dpc_copy_d2h": (_i, [_vp, _vp, _vp, ctypes.c_size_t]),
    "dpc_copy_h2d_sync": (_i, [_vp, _vp, _vp, ctypes.c_size_t]),
    "dpc_copy_d2h_sync": (_i, [_vp, _vp, _vp, ctypes.c_size_t]),
    "dpc_alloc_host": (_i, [_vp, ctypes.c_size_t, ctypes.POINTER(_vp)]),
    "dpc_free_host": (_i, [_vp, _vp]),
    "dpc_sync": (_i, [_vp]),
    "dpc_gather_rows": (_i, [_vp, _vp, _vp, _i64, _i, _i64, _vp]),
    "dpc_graph_begin": (_i, [_vp, _i]),
    "dpc_graph_end": (_i, [_vp, _i]),
    "dpc_graph_launch": (_i, [_vp, _i]),
    "dpc_graph_drop": (_i, [_vp, _i]),
    "dpc_plan_create": (_i, [_vp, _vp, _i, _i, ctypes.POINTER(_vp)]),
    "dpc_plan_update": (_i, [_vp, _vp, _i]),
    "dpc_plan_destroy": (_i, [_vp]),
    "dpc_plan_set_terminal_error": (_i, [_vp, _vp]),
    "dpc_plan_set_chain_trace": (_i, [_vp, _vp]),
    "dpc_plan_tensor_run": (_i, [_vp, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "dpc_plan_describe": (_i, [_vp, _cp, _i]),
    "dpc_plan_invalidate": (_i, [_vp, _i, _i, _i]),
    "dpc_plan_sync_operands": (_i, [_vp]),
    "dpc_plan_set_wait_limit": (_i, [_vp, ctypes.c_double, _i]),
    "dpc_forward": (_i, [_vp, _i, _i, _i]),
    "dpc_project_forward": (_i, [_vp, _i, _i, _i]),
    "dpc_project_forward_ex": (_i, [_vp, _i, _i, _i, _i]),
    "dpc_error": (_i, [_vp, _i, _i]),
    "dpc_feedback_error": (_i, [_vp, _i, _i]),
    "dpc_update_state": (_i, [_vp, _i, _i]),
    "dpc_epc_reconstruct": (_i, [_vp, _i]),
    "dpc_epc_adjoint": (_i, [_vp, _i, _i, _f, _i]),
    "dpc_relax": (_i, [_vp, _i]),
    "dpc_direct_feedback": (_i, [_vp, _i, _i, _i]),
    "dpc_update_weights": (_i, [_vp, _i, _i, _i]),
    "dpc_weight_gradients": (_i, [_vp, _i, _i, _i]),
    "dpc_apply_gradients": (_i, [_vp, _i, _i, _i, _i, _i]),
    "dpc_error_energy_static": (_i, [_vp, _vp, _vp, _vp, _i64, _vp]),
    "dpc_energy_reset": (_i, [_vp]),
    "dpc_energy_read": (_i, [_vp, ctypes.POINTER(ctypes.c_double)]),
    "dpcn_create": (_i, [_i, _i, _i, ctypes.POINTER(_vp)]),
    "dpcn_destroy": (_i, [_vp]),
    "dpcn_add_layer": (_i, [_vp, _i, _i, _i, _f, _f, _f, _f, _i]),
    "dpcn_set_option": (_i, [_vp, _cp, _i, _f]),
    "dpcn_compile": (_i, [_vp]),
    "dpcn_num_layers": (_i, [_vp]),
    "dpcn_tensor_size": (_i64, [_vp, _i, _cp]),
    "dpcn_get_tensor": (_i, [_vp, _i, _cp, c_f32p, _i64]),
    "dpcn_set_tensor": (_i, [_vp, _i, _cp, c_f32p, _i64]),
    "dpcn_get_counter": (_i, [_vp, _i, _cp, ctypes.POINTER(ctypes.c_int32)]),
    "dpcn_set_counter": (_i, [_vp, _i, _cp, ctypes.c_int32]),
    "dpcn_state_dict_size": (_i, [_vp]),
    "dpcn_state_dict_entry": (_i, [_vp, _i, ctypes.POINTER(_i), _cp, _i, ctypes.POINTER(_i64),
                                   ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i)]),
    "dpcn_tensor_ptr": (_i, [_vp, _i, _cp, ctypes.POINTER(_vp), ctypes.POINTER(_i64)]),
    "dpcn_randomize": (_i, [_vp, ctypes.c_uint32]),
    "dpcn_train_step": (_i, [_vp, c_f32p, _i64, c_f32p, _i64, _i, c_f32p]),
    "dpcn_train_step_device": (_i, [_vp, _vp, _i64, _vp, _i64, _i, c_f32p]),
    "dpcn_train_step_mode": (_i, [_vp, _i, c_f32p, _i64, c_f32p, _i64, _i, c_f32p]),
    "dpcn_predict": (_i, [_vp, c_f32p, _i64, _i, _i, c_f32p, _i64]),
    "dpcn_reset_state": (_i, [_vp]),
    "dpcn_context": (_vp, [_vp]),
    "dpcn_plan": (_vp, [_vp]),
    "dpcn_set_gradient_sync": (_i, [_vp, _vp, _vp, _i]),
    "dpcn_launch_count": (_i64, [_vp]),
    "dpcn_train_step_flops": (ctypes.c_double, [_vp, _i]),
    "dpc_conv_plan_create": (_i, [_vp, _vp, _i, _i, ctypes.POINTER(_vp)]),
    "dpc_conv_plan_update": (_i, [_vp, _vp, _i]),
    "dpc_conv_plan_destroy": (_i, [_vp]),
    "dpc_conv_forward": (_i, [_vp, _i, _i]),
    "dpc_conv_update_state": (_i, [_vp, _i]),
    "dpc_conv_gate_with_prediction": (_i, [_vp, _i]),
    "dpc_conv_update_weights": (_i, [_vp, _i, _i]),
    "dpc_conv_energy_reset": (_i, [_vp]),
    "dpc_conv_energy_read": (_i, [_vp, ctypes.POINTER(ctypes.c_double)]),
    "dpcn_conv_create": (_i, [_i, _i, ctypes.POINTER(_vp)]),
    "dpcn_conv_destroy": (_i, [_vp]),
    "dpcn_conv_add_layer": (_i, [_vp] + [_i] * 10 + [_f] * 3 + [_i]),
    "dpcn_conv_set_option": (_i, [_vp, _cp, _i, _f]),
    "dpcn_conv_compile": (_i, [_vp]),
    "dpcn_conv_num_layers": (_i, [_vp]),
    "dpcn_conv_layer_shape": (_i, [_vp, _i, ctypes.POINTER(_i)]),
    "dpcn_conv_tensor_size": (_i64, [_vp, _i, _cp]),
    "dpcn_conv_get_tensor": (_i, [_vp, _i, _cp, c_f32p, _i64]),
    "dpcn_conv_set_tensor": (_i, [_vp, _i, _cp, c_f32p, _i64]),
    "dpcn_conv_randomize": (_i, [_vp, ctypes.c_uint32]),
    "dpcn_conv_train_step": (_i, [_vp, _vp, _i64, _vp, _i64, _i, _i, _i, c_f32p]),
    "dpcn_conv_predict": (_i, [_vp, c_f32p, _i64, _i, _i, c_f32p, _i64]),
    "dpcn_conv_context": (_vp, [_vp]),
    "dpcn_conv_plan": (_vp, [_vp]),
    "dpcn_conv_launch_count": (_i64, [_vp]),
}

_lib = None


class DeepityError(RuntimeError):
    """A dpc_* / dpcn_* call returned a negative status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"deepity_b200 error {status}: {message}")
        self.status = status


def load():
    """Load the shared library (once) and attach the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m deepity_b200.build` "
            "(needs nvcc; there is no pure-Python or CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> int:
    if status < 0:
        raise DeepityError(status, load().dpc_last_error().decode(errors="replace"))
    return status

"""ctypes binding of the compiled reference CPU path (``oracle/_ref/libdeepity_ref.so``).

Test infrastructure only.  The library is built by ``oracle/build_ref.py`` from the
reference checkout; its flat C interface is ``oracle/ref_driver.cpp``.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "libdeepity_ref.so")

KIND = {"simple": 0, "dkp": 1, "full": 2}
# Forward enumerators of Deep::ActivationType (include/deepity/utils/ActivationType.h:15-32).
ACT = {"relu": 0, "gelu": 2, "sigmoid": 4, "esigmoid": 6, "tanh": 8, "linear": 10, "hard_tanh": 12}
OPT = {"SGD": 0, "ADAM": 1, "ADAMW": 2}

_lib = None


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(_LIB_PATH)
        f32p = ctypes.POINTER(ctypes.c_float)
        L.ref_create.restype = ctypes.c_void_p
        L.ref_create.argtypes = [ctypes.c_int, ctypes.c_int]
        L.ref_create_on_gpu.restype = ctypes.c_void_p
        L.ref_create_on_gpu.argtypes = [ctypes.c_int, ctypes.c_int]
        L.ref_destroy.argtypes = [ctypes.c_void_p]
        L.ref_add_layer.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                    ctypes.c_float, ctypes.c_int]
        L.ref_set_option.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int,
                                     ctypes.c_float]
        L.ref_compile.argtypes = [ctypes.c_void_p]
        L.ref_num_layers.argtypes = [ctypes.c_void_p]
        L.ref_tensor_size.restype = ctypes.c_int64
        L.ref_tensor_size.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p]
        L.ref_get_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, f32p,
                                     ctypes.c_int64]
        L.ref_set_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, f32p,
                                     ctypes.c_int64]
        L.ref_train_step.restype = ctypes.c_float
        L.ref_train_step.argtypes = [ctypes.c_void_p, f32p, ctypes.c_int64, f32p,
                                     ctypes.c_int64, ctypes.c_int]
        L.ref_train_step_with_projection.restype = ctypes.c_float
        L.ref_train_step_with_projection.argtypes = [ctypes.c_void_p, f32p, ctypes.c_int64, f32p,
                                                     ctypes.c_int64, ctypes.c_int, ctypes.c_int]
        L.ref_predict.argtypes = [ctypes.c_void_p, f32p, ctypes.c_int64, ctypes.c_int,
                                  ctypes.c_int, f32p, ctypes.c_int64]
        L.ref_phase.restype = ctypes.c_float
        L.ref_phase.argtypes = [ctypes.c_void_p, ctypes.c_char_p, f32p, ctypes.c_int64]
        L.ref_omp_threads.restype = ctypes.c_int
        L.ref_num_procs.restype = ctypes.c_int
        L.ref_blas_config.restype = ctypes.c_char_p
        L.ref_backend_matmul.argtypes = [ctypes.c_int] * 6 + [ctypes.c_float, f32p, ctypes.c_int64,
                                         ctypes.c_int, f32p, ctypes.c_int64, ctypes.c_int,
                                         ctypes.c_float, f32p, ctypes.c_int64, ctypes.c_int,
                                         ctypes.c_int]
        L.ref_blas_threads.restype = ctypes.c_int
        L.ref_set_threads.argtypes = [ctypes.c_int]
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


class RefNet:
    """One reference network (``kind`` in 'simple' | 'dkp' | 'full') on the CPU backend.

    ``sizes`` lists the layer widths, e.g. [784, 256, 10]; one weight layer is added
    per consecutive pair plus the weight-less terminal layer, the way the Python
    wrappers of the reference build their networks (deepity/DKPPCN.py:101-148).
    """

    def __init__(self, kind: str, sizes, batch: int, *, lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0,
                 act="tanh", last_act=None, options=None, device="cpu"):
        self.kind, self.sizes, self.batch = kind, list(sizes), batch
        L = lib()
        if device == "cpu":
            self.h = L.ref_create(KIND[kind], batch)
        else:
            # DEVICE_GPU: the reference's loader looks for libDeepityCUDA.so beside this library
            self.h = L.ref_create_on_gpu(KIND[kind], batch)
            if not self.h:
                raise RuntimeError("the reference could not load a GPU backend plugin")
        ts = self.sizes[-1]
        n_w = len(self.sizes) - 1
        for i in range(n_w):
            a = act if (i + 1 < n_w or last_act is None) else last_act
            L.ref_add_layer(self.h, self.sizes[i], self.sizes[i + 1], ts, lr, ir, fl, lmbda, ACT[a])
        L.ref_add_layer(self.h, ts, 0, ts, lr, ir, fl, lmbda, ACT["linear"])
        for name, val in (options or {}).items():
            self.set_option(name, val)
        if L.ref_compile(self.h) != 0:
            raise RuntimeError("reference Compile() failed")

    def set_option(self, name, val):
        if isinstance(val, str):
            iv, fv = OPT[val], 0.0
        elif isinstance(val, tuple):
            iv, fv = int(val[0]), float(val[1])
        elif isinstance(val, float):
            iv, fv = 1, val
        else:
            iv, fv = int(val), 0.0
        if lib().ref_set_option(self.h, name.encode(), iv, fv) != 0:
            raise ValueError(f"option {name!r} rejected by the reference driver")

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_destroy(self.h)
            self.h = None

    @property
    def num_layers(self) -> int:
        return lib().ref_num_layers(self.h)

    def get(self, layer: int, name: str) -> np.ndarray:
        n = lib().ref_tensor_size(self.h, layer, name.encode())
        out = np.empty(n, dtype=np.float32)
        if n and lib().ref_get_tensor(self.h, layer, name.encode(), _ptr(out), n) != 0:
            raise KeyError((layer, name))
        return out

    def set(self, layer: int, name: str, value) -> None:
        v = np.ascontiguousarray(value, dtype=np.float32).ravel()
        if lib().ref_set_tensor(self.h, layer, name.encode(), _ptr(v), v.size) != 0:
            raise KeyError((layer, name, v.size))

    def train_step(self, x, y, T: int) -> float:
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        y = np.ascontiguousarray(y, dtype=np.float32).ravel()
        return float(lib().ref_train_step(self.h, _ptr(x), x.size, _ptr(y), y.size, T))

    def train_step_with_projection(self, x, y, T: int, energy=True) -> float:
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        y = np.ascontiguousarray(y, dtype=np.float32).ravel()
        return float(lib().ref_train_step_with_projection(self.h, _ptr(x), x.size, _ptr(y),
                                                          y.size, T, int(energy)))

    def predict(self, x, T: int, with_projection=False) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        out = np.empty(self.batch * self.sizes[-1], dtype=np.float32)
        if lib().ref_predict(self.h, _ptr(x), x.size, T, int(with_projection), _ptr(out),
                             out.size) != 0:
            raise RuntimeError("reference Predict() size mismatch")
        return out.reshape(self.batch, self.sizes[-1])

    def phase(self, op: str, data=None) -> float:
        if data is None:
            return float(lib().ref_phase(self.h, op.encode(), None, 0))
        d = np.ascontiguousarray(data, dtype=np.float32).ravel()
        return float(lib().ref_phase(self.h, op.encode(), _ptr(d), d.size))


def host_info() -> dict:
    L = lib()
    return {"omp_threads": L.ref_omp_threads(), "nproc": L.ref_num_procs(),
            "blas_threads": L.ref_blas_threads(), "blas": L.ref_blas_config().decode()}


def backend_matmul(device: str, trans_a: bool, trans_b: bool, M: int, N: int, K: int, alpha: float,
                   A: np.ndarray, lda: int, B: np.ndarray, ldb: int, beta: float, C: np.ndarray,
                   ldc: int, allow_tf32=None) -> np.ndarray:
    """C = alpha*op(A)*op(B) + beta*C through IComputeBackend::MatMul of the reference's CPU backend
    (device 'cpu') or of whatever GPU plugin its loader finds ('gpu'); returns the new C."""
    a = np.ascontiguousarray(A, dtype=np.float32).ravel()
    b = np.ascontiguousarray(B, dtype=np.float32).ravel()
    c = np.ascontiguousarray(C, dtype=np.float32).ravel().copy()
    rc = lib().ref_backend_matmul(int(device != "cpu"), int(trans_a), int(trans_b), M, N, K, alpha,
                                  _ptr(a), a.size, lda, _ptr(b), b.size, ldb, beta, _ptr(c), c.size,
                                  ldc, -1 if allow_tf32 is None else int(allow_tf32))
    if rc != 0:
        raise RuntimeError(f"backend MatMul failed ({rc})")
    return c


def set_threads(n: int) -> None:
    """Cap the OpenMP / OpenBLAS thread count of the compiled reference (after its own
    DynamicThread policy has run once, i.e. after the first train step)."""
    lib().ref_set_threads(int(n))


class RefConvNet:
    """The reference's CPU SimpleConvPCNetwork (oracle/ref_conv_driver.cpp).

    ``layers``: list of dicts(inC, outC, H, W, kH, kW, sH, sW, pH, pW, act); the last one has
    outC = 0 (the terminal layer)."""

    def __init__(self, layers, batch, lr, ir, lmbda, optimizer="SGD", center_weights=False,
                 device="cpu"):
        L = lib()
        f32p = ctypes.POINTER(ctypes.c_float)
        L.refc_create.restype = ctypes.c_void_p
        L.refc_create.argtypes = [ctypes.c_int]
        L.refc_destroy.argtypes = [ctypes.c_void_p]
        L.refc_add_layer.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 10 + \
            [ctypes.c_float] * 3 + [ctypes.c_int]
        L.refc_set_option.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int,
                                      ctypes.c_float]
        L.refc_compile.argtypes = [ctypes.c_void_p]
        L.refc_tensor_size.restype = ctypes.c_int64
        L.refc_tensor_size.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p]
        L.refc_get_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, f32p,
                                      ctypes.c_int64]
        L.refc_set_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, f32p,
                                      ctypes.c_int64]
        L.refc_train_step.restype = ctypes.c_float
        L.refc_train_step.argtypes = [ctypes.c_void_p, f32p, ctypes.c_int64, f32p, ctypes.c_int64,
                                      ctypes.c_int, ctypes.c_int]
        L.refc_predict.argtypes = [ctypes.c_void_p, f32p, ctypes.c_int64, ctypes.c_int,
                                   ctypes.c_int, f32p, ctypes.c_int64]
        self.L, self.batch, self.layers = L, batch, layers
        if device == "cpu":
            self.h = ctypes.c_void_p(L.refc_create(batch))
        else:
            # the reference's own device path, on whatever libDeepityCUDA.so its loader finds
            L.refc_create_on_gpu.restype = ctypes.c_void_p
            L.refc_create_on_gpu.argtypes = [ctypes.c_int]
            self.h = ctypes.c_void_p(L.refc_create_on_gpu(batch))
            if not self.h:
                raise RuntimeError("the reference could not create its GPU backend")
        for d in layers:
            L.refc_add_layer(self.h, d["inC"], d["outC"], d["H"], d["W"], d["kH"], d["kW"],
                             d["sH"], d["sW"], d["pH"], d["pW"], lr, ir, lmbda, ACT[d["act"]])
        L.refc_set_option(self.h, b"optimizer", OPT[optimizer], 0.0)
        L.refc_compile(self.h)
        L.refc_set_option(self.h, b"center_weights", int(center_weights), 0.0)

    def __del__(self):
        if getattr(self, "h", None):
            self.L.refc_destroy(self.h)
            self.h = None

    def get(self, layer, name):
        n = self.L.refc_tensor_size(self.h, layer, name.encode())
        if n < 0:
            raise KeyError((layer, name))
        out = np.empty(n, dtype=np.float32)
        self.L.refc_get_tensor(self.h, layer, name.encode(), _ptr(out), n)
        return out

    def set(self, layer, name, value):
        v = np.ascontiguousarray(value, dtype=np.float32).ravel()
        if self.L.refc_set_tensor(self.h, layer, name.encode(), _ptr(v), v.size) != 0:
            raise KeyError((layer, name, v.size))

    def train_step(self, x, y, T, with_projection=False):
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        y = np.ascontiguousarray(y, dtype=np.float32).ravel()
        return float(self.L.refc_train_step(self.h, _ptr(x), x.size, _ptr(y), y.size, T,
                                            int(with_projection)))

    def predict(self, x, T, with_projection=False):
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        last = self.layers[-1]
        out = np.empty(self.batch * last["inC"] * last["H"] * last["W"], dtype=np.float32)
        if self.L.refc_predict(self.h, _ptr(x), x.size, T, int(with_projection), _ptr(out),
                               out.size) != 0:
            raise RuntimeError("reference Predict() size mismatch")
        return out

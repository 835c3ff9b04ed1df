"""``SimpleConvolutionalPCN``: the reference's convolutional predictive-coding network
(``deepity/SimpleConvolutionalPCN.py``) over the ``dpcn_conv_*`` C ABI.

Same architecture DSL (``Convolution`` + activations, closed by ``Convolution(0, 1, 1)``),
same ``configure`` keywords, ``train_step`` / ``train_step_with_projection`` / ``predict`` /
``predict_with_projection`` / ``fit``.  Tensors are NCHW, weights ``[out_channels,
in_channels*kernel_h*kernel_w]`` as the reference's state dict exposes them.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from . import _lib
from .layer import ACT_IDS, OPT_IDS, Activation, Convolution


def _f32(a) -> np.ndarray:
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32).ravel()


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class ConvLayerView:
    """One layer of a compiled network: geometry and tensors (copies)."""

    def __init__(self, net, index, in_shape, out_shape, row_len):
        self._net, self.index = net, index
        self.in_channels, self.in_height, self.in_width = in_shape
        self.out_channels, self.out_height, self.out_width = out_shape
        self.row_len = row_len

    @property
    def weights(self):
        return self._net.get_tensor(self.index, "W").reshape(self.out_channels, self.row_len)

    @property
    def biases(self):
        return self._net.get_tensor(self.index, "b")

    @property
    def beliefs(self):
        return self._net.get_tensor(self.index, "z").reshape(
            self._net.batch_size, self.in_channels, self.in_height, self.in_width)

    @property
    def errors(self):
        return self._net.get_tensor(self.index, "e").reshape(
            self._net.batch_size, self.in_channels, self.in_height, self.in_width)

    def set_weights(self, w):
        self._net.set_tensor(self.index, "W", w)

    def set_biases(self, b):
        self._net.set_tensor(self.index, "b", b)


class SimpleConvolutionalPCN:
    def __init__(self, *architecture, input_shape, batch_size: Optional[int] = None,
                 device="cuda"):
        self.architecture = architecture
        self.input_shape = tuple(int(v) for v in input_shape)
        self.batch_size = 64 if batch_size is None else int(batch_size)
        self.device = device
        self._configured = False
        self._h = ctypes.c_void_p()
        self.layers: list[ConvLayerView] = []
        self._validate_architecture()
        dev = 0
        if isinstance(device, str) and ":" in device:
            dev = int(device.split(":")[1])
        elif isinstance(device, int):
            dev = device
        if isinstance(device, str) and device.split(":")[0] not in ("cuda", "gpu"):
            raise ValueError(f"SimpleConvolutionalPCN: device {device!r} is not supported; this "
                             "build runs on CUDA devices only (no CPU backend)")
        self._lib = _lib.load()
        _lib.check(self._lib.dpcn_conv_create(self.batch_size, dev, ctypes.byref(self._h)))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and h.value:
            self._lib.dpcn_conv_destroy(h)
            self._h = ctypes.c_void_p()

    # deepity/SimpleConvolutionalPCN.py:44-67
    def _validate_architecture(self) -> None:
        if not self.architecture:
            raise ValueError("Architecture cannot be empty.")
        if not isinstance(self.architecture[0], Convolution):
            raise ValueError("Architecture must begin with Convolution.")
        previous_was_activation = False
        for layer in self.architecture:
            if isinstance(layer, Convolution):
                previous_was_activation = False
            elif isinstance(layer, Activation):
                if previous_was_activation:
                    raise ValueError("Consecutive activation functions are not allowed.")
                previous_was_activation = True
            else:
                raise TypeError(f"Unsupported architecture object: {type(layer).__name__}")

    # deepity/SimpleConvolutionalPCN.py:69-107
    def _build_backend(self) -> None:
        c, h, w = self.input_shape
        arch = self.architecture
        idx = 0
        for i, layer in enumerate(arch):
            if not isinstance(layer, Convolution):
                continue
            act = "linear"
            if i + 1 < len(arch) and isinstance(arch[i + 1], Activation):
                act = arch[i + 1].to_string()
            _lib.check(self._lib.dpcn_conv_add_layer(
                self._h, c, layer.out_channels, h, w, layer.kernel_h, layer.kernel_w,
                layer.stride_h, layer.stride_w, layer.pad_h, layer.pad_w, self._learning_rate,
                self._inference_rate, self._lambda, ACT_IDS[act]))
            shape = (ctypes.c_int * 4)()
            _lib.check(self._lib.dpcn_conv_layer_shape(self._h, idx, shape))
            self.layers.append(ConvLayerView(self, idx, (c, h, w), tuple(shape[:3]), shape[3]))
            idx += 1
            if layer.out_channels > 0:
                c, h, w = shape[0], shape[1], shape[2]

    def configure(self, learning_rate: float = 1e-6, inference_rate: float = 0.1,
                  lmbda: float = 1e-2, optimizer: str = "SGD", center_weights: bool = False,
                  seed: Optional[int] = None):
        if self._configured:
            raise RuntimeError("configure() may be called only once")
        self._learning_rate, self._inference_rate = float(learning_rate), float(inference_rate)
        self._lambda, self._optimizer = float(lmbda), optimizer
        self._build_backend()
        self._option("optimizer", OPT_IDS[optimizer.upper()])
        _lib.check(self._lib.dpcn_conv_compile(self._h))
        self.randomize_weights(seed)
        self._configured = True
        self.set_center_weights(center_weights)
        return self

    def _option(self, name, ivalue=0, fvalue=0.0):
        _lib.check(self._lib.dpcn_conv_set_option(self._h, name.encode(), int(ivalue), float(fvalue)))

    def _require_configured(self):
        if not self._configured:
            raise RuntimeError("SimpleConvolutionalPCN must be configured before use. "
                               "Call configure() first.")

    def randomize_weights(self, seed: Optional[int] = None):
        if seed is None:
            seed = int(np.random.SeedSequence().generate_state(1)[0])
        _lib.check(self._lib.dpcn_conv_randomize(self._h, seed & 0xFFFFFFFF))

    def set_center_weights(self, enabled: bool):
        self._require_configured()
        self._center_weights = bool(enabled)
        self._option("center_weights", int(enabled))

    def set_learning_rate(self, lr: float):
        self._require_configured()
        self._option("learning_rate", fvalue=lr)
        self._learning_rate = float(lr)

    def set_inference_rate(self, ir: float):
        self._require_configured()
        self._option("inference_rate", fvalue=ir)
        self._inference_rate = float(ir)

    def set_lambda(self, lmbda: float):
        self._require_configured()
        self._option("lambda", fvalue=lmbda)
        self._lambda = float(lmbda)

    def set_optimizer(self, optimizer: str):
        self._require_configured()
        self._option("optimizer", OPT_IDS[optimizer.upper()])
        self._optimizer = optimizer

    def set_use_graph(self, enabled: bool):
        self._option("use_graph", int(enabled))

    # ---- tensors ---------------------------------------------------------------------
    def get_tensor(self, layer: int, name: str) -> np.ndarray:
        n = self._lib.dpcn_conv_tensor_size(self._h, layer, name.encode())
        if n < 0:
            raise KeyError(f"layer {layer} has no tensor {name!r}")
        out = np.empty(n, dtype=np.float32)
        _lib.check(self._lib.dpcn_conv_get_tensor(self._h, layer, name.encode(),
                                                  out.ctypes.data_as(_lib.c_f32p), n))
        return out

    def set_tensor(self, layer: int, name: str, value) -> None:
        v = _f32(value)
        _lib.check(self._lib.dpcn_conv_set_tensor(self._h, layer, name.encode(),
                                                  v.ctypes.data_as(_lib.c_f32p), v.size))

    # ---- compute ---------------------------------------------------------------------
    def _train(self, X, Y, steps, with_projection):
        self._require_configured()
        x, y = _f32(X), _f32(Y)
        e = ctypes.c_float()
        _lib.check(self._lib.dpcn_conv_train_step(self._h, _ptr(x), x.size, _ptr(y), y.size,
                                                  int(steps), int(with_projection), 0,
                                                  ctypes.byref(e)))
        return float(e.value)

    def train_step(self, X, Y, steps: int) -> float:
        return self._train(X, Y, steps, False)

    def train_step_with_projection(self, X, Y, steps: int) -> float:
        return self._train(X, Y, steps, True)

    def train_step_device(self, x_dev, y_dev, steps: int, with_projection: bool = False) -> float:
        """Inputs already on this GPU (CUDA torch tensors)."""
        self._require_configured()
        e = ctypes.c_float()
        _lib.check(self._lib.dpcn_conv_train_step(
            self._h, ctypes.c_void_p(x_dev.data_ptr()), x_dev.numel(),
            ctypes.c_void_p(y_dev.data_ptr()), y_dev.numel(), int(steps), int(with_projection), 1,
            ctypes.byref(e)))
        return float(e.value)

    def _predict(self, X, steps, with_projection):
        self._require_configured()
        x = _f32(X)
        last = self.layers[-1]
        n = self.batch_size * last.in_channels * last.in_height * last.in_width
        out = np.empty(n, dtype=np.float32)
        _lib.check(self._lib.dpcn_conv_predict(self._h, x.ctypes.data_as(_lib.c_f32p), x.size,
                                               int(steps), int(with_projection),
                                               out.ctypes.data_as(_lib.c_f32p), n))
        return out.reshape(self.batch_size, -1)

    def predict(self, X, steps: int):
        return self._predict(X, steps, False)

    def predict_with_projection(self, X, steps: int):
        return self._predict(X, steps, True)

    def fit(self, X, Y, epochs: int, steps: int, initial_lr: Optional[float] = None,
            decay_rate: float = 1.0, shuffle: bool = True):
        """Epoch loop of ``deepity/utils.py:19-143`` without the progress bars."""
        self._require_configured()
        X = np.asarray(X, dtype=np.float32)
        Y = np.asarray(Y, dtype=np.float32)
        n, bsz = len(X), self.batch_size
        if n == 0:
            raise ValueError("Training data cannot be empty.")
        if n % bsz != 0:
            raise ValueError(f"Number of samples ({n}) must be divisible by batch_size ({bsz}).")
        if initial_lr is None:
            initial_lr = self._learning_rate
        for epoch in range(epochs):
            self.set_learning_rate(initial_lr * (decay_rate ** epoch))
            idx = np.random.permutation(n) if shuffle else np.arange(n)
            for b in range(n // bsz):
                sel = idx[b * bsz:(b + 1) * bsz]
                self.train_step(X[sel], Y[sel], steps)
        return self

    @property
    def launch_count(self) -> int:
        return int(self._lib.dpcn_conv_launch_count(self._h))

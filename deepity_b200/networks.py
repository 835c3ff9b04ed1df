"""Python surface: ``SimplePCN`` / ``DKPPCN`` / ``FullPCN``.

Same constructor DSL, ``configure(...)`` keywords, ``train_step`` / ``predict`` / ``fit``
and per-layer ``weights`` / ``biases`` / ``psi`` / ``beliefs`` / ``errors`` accessors as the
reference's ``deepity/SimplePCN.py``, ``DKPPCN.py`` and ``FullPCN.py``; underneath, every
call goes through the ``dpcn_*`` C ABI of ``libdeepity_b200.so`` to the sm_100a kernels.
Inputs are numpy arrays, or anything ``numpy.asarray`` understands; CUDA ``torch`` tensors
are taken zero-copy by ``train_step_device``.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib
from .layer import ACT_IDS, OPT_IDS, Activation, Layer, Linear

KIND_SIMPLE, KIND_DKP, KIND_FULL = 0, 1, 2


def _f32(a) -> np.ndarray:
    if hasattr(a, "detach") and hasattr(a, "cpu"):  # torch tensor
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32).ravel()


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_lib.c_f32p)


class LayerView:
    """One layer of a configured network (reference: ``net.layers[i]``)."""

    def __init__(self, net: "_Network", index: int, size: int, next_size: int):
        self._net, self.index, self.size, self.next_size = net, index, size, next_size

    def _get(self, name, shape):
        return self._net.get_tensor(self.index, name).reshape(shape)

    @property
    def weights(self):
        return self._get("W", (self.next_size, self.size))

    @property
    def biases(self):
        return self._get("b", (self.next_size,))

    @property
    def psi(self):
        return self._get("Psi", (self.size, self._net.terminal_size))

    @property
    def beliefs(self):
        return self._get("z", (self._net.batch_size, self.size))

    @property
    def errors(self):
        return self._get("e", (self._net.batch_size, self.size))

    @property
    def mu(self):
        return self._get("mu", (self._net.batch_size, self.next_size))

    def set_weights(self, w):
        self._net.set_tensor(self.index, "W", w)

    def set_biases(self, b):
        self._net.set_tensor(self.index, "b", b)

    def set_psi(self, p):
        self._net.set_tensor(self.index, "Psi", p)


class _Network:
    KIND = KIND_DKP
    NAME = "network"

    def __init__(self, *architecture, batch_size: Optional[int] = None, device="cuda"):
        self.architecture = architecture
        self.batch_size = 64 if batch_size is None else int(batch_size)
        self.device = device
        self.default_inference_steps = 1
        self._configured = False
        self._h = ctypes.c_void_p()
        self._validate_architecture()
        dev = 0
        if isinstance(device, str) and ":" in device:
            dev = int(device.split(":")[1])
        elif isinstance(device, int):
            dev = device
        if isinstance(device, str) and device.split(":")[0] not in ("cuda", "gpu"):
            raise ValueError(f"{self.NAME}: device {device!r} is not supported; this build runs on "
                             "CUDA devices only (no CPU backend)")
        self._lib = _lib.load()
        self._device_index = dev
        _lib.check(self._lib.dpcn_create(self.KIND, self.batch_size, dev, ctypes.byref(self._h)))
        self.layers: list[LayerView] = []

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and h.value:
            self._lib.dpcn_destroy(h)
            self._h = ctypes.c_void_p()

    # ---- architecture (deepity/DKPPCN.py:66-148) -------------------------------------
    def _validate_architecture(self) -> None:
        arch = self.architecture
        if not arch:
            raise ValueError(f"{self.NAME} requires at least one layer.")
        if not isinstance(arch[0], Linear):
            raise TypeError("Architecture must begin with a Linear layer.")
        if not isinstance(arch[-1], (Linear, Activation)):
            raise TypeError("Network architecture must end with a Linear or Activation layer.")
        prev = None
        for layer in arch:
            if isinstance(layer, Linear):
                if prev is not None and prev.out_n != layer.in_n:
                    raise ValueError(f"Layer dimensions do not match: {prev.out_n} != {layer.in_n}.")
                prev = layer
            elif isinstance(layer, Activation):
                if prev is None:
                    raise ValueError("An activation cannot appear before the first Linear layer.")
            else:
                raise TypeError(f"Unsupported architecture element: {type(layer).__name__}.")

    @property
    def terminal_size(self) -> int:
        for layer in reversed(self.architecture):
            if isinstance(layer, Linear):
                return layer.out_n
        raise RuntimeError("No terminal Linear layer found.")

    def _linears(self):
        arch = self.architecture
        for i, layer in enumerate(arch):
            if isinstance(layer, Linear):
                act = "linear"
                if i + 1 < len(arch) and isinstance(arch[i + 1], Activation):
                    act = arch[i + 1].to_string()
                yield layer, act

    def _build_backend(self, lr, ir, fl, lmbda) -> None:
        ts = self.terminal_size
        idx = 0
        for layer, act in self._linears():
            _lib.check(self._lib.dpcn_add_layer(self._h, layer.in_n, layer.out_n, ts, lr, ir, fl,
                                                lmbda, ACT_IDS[act]))
            self.layers.append(LayerView(self, idx, layer.in_n, layer.out_n))
            idx += 1
        _lib.check(self._lib.dpcn_add_layer(self._h, ts, 0, ts, lr, ir, fl, lmbda,
                                            ACT_IDS["linear"]))
        self.layers.append(LayerView(self, idx, ts, 0))

    def _option(self, name: str, ivalue: int = 0, fvalue: float = 0.0) -> None:
        _lib.check(self._lib.dpcn_set_option(self._h, name.encode(), int(ivalue), float(fvalue)))

    def _require_configured(self) -> None:
        if not self._configured:
            raise RuntimeError(f"{self.NAME} has not been configured. "
                               "Call net.configure(...) before training or prediction.")

    # ---- tensors ---------------------------------------------------------------------
    def get_tensor(self, layer: int, name: str) -> np.ndarray:
        n = self._lib.dpcn_tensor_size(self._h, layer, name.encode())
        if n <= 0:
            raise KeyError(f"layer {layer} has no tensor {name!r}")
        out = np.empty(n, dtype=np.float32)
        _lib.check(self._lib.dpcn_get_tensor(self._h, layer, name.encode(), _ptr(out), n))
        return out

    def set_tensor(self, layer: int, name: str, value) -> None:
        v = _f32(value)
        _lib.check(self._lib.dpcn_set_tensor(self._h, layer, name.encode(), _ptr(v), v.size))

    def tensor_ptr(self, layer: int, name: str) -> int:
        p = ctypes.c_void_p()
        stride = ctypes.c_int64()
        _lib.check(self._lib.dpcn_tensor_ptr(self._h, layer, name.encode(), ctypes.byref(p),
                                             ctypes.byref(stride)))
        return p.value

    # ---- setters (deepity/DKPPCN.py:218-262) -------------------------------------------
    def set_optimizer(self, optimizer: str) -> None:
        self._option("optimizer", OPT_IDS[optimizer.upper()])
        self._optimizer = optimizer

    def set_center_weights(self, enabled: bool) -> None:
        self._option("center_weights", int(bool(enabled)))

    def set_learning_rate(self, learning_rate: float) -> None:
        self._option("learning_rate", 0, learning_rate)
        self._learning_rate = learning_rate

    def set_inference_rate(self, inference_rate: float) -> None:
        self._option("inference_rate", 0, inference_rate)
        self._inference_rate = inference_rate

    def set_precision(self, precision: str) -> None:
        """'fp32' (parity with the CPU reference at 1e-4), 'tf32' (one tensor-core pass, 1e-2) or
        'mixed' (fp32 state path, tf32 gradient products when all weight optimizers are SGD, 1e-3)."""
        self._option("precision", {"fp32": 0, "tf32": 1, "mixed": 2}[precision])

    def set_use_graph(self, enabled: bool) -> None:
        self._option("use_graph", int(bool(enabled)))

    def randomize_weights(self, seed: Optional[int] = None, dist: str = "normal") -> None:
        if seed is None:
            seed = int(np.random.SeedSequence().generate_state(1)[0])
        _lib.check(self._lib.dpcn_randomize(self._h, seed & 0xFFFFFFFF))

    # ---- compute ---------------------------------------------------------------------
    def _train(self, mode: int, X, Y, steps: int) -> float:
        self._require_configured()
        x, y = _f32(X), _f32(Y)
        e = ctypes.c_float()
        _lib.check(self._lib.dpcn_train_step_mode(self._h, mode, _ptr(x), x.size, _ptr(y), y.size,
                                                  int(steps), ctypes.byref(e)))
        return float(e.value)

    def train_step(self, X, Y, inference_steps: int = 1) -> float:
        """One training step on one batch; returns the network energy."""
        return self._train(0, X, Y, inference_steps)

    def train_step_device(self, x_dev, y_dev, inference_steps: int = 1, read_energy=True):
        """Same with inputs already resident on this GPU (CUDA torch tensors or raw device
        addresses); with ``read_energy=False`` the call only enqueues work."""
        self._require_configured()

        def addr(t):
            return (t.data_ptr(), t.numel()) if hasattr(t, "data_ptr") else t

        (xp, xn), (yp, yn) = addr(x_dev), addr(y_dev)
        e = ctypes.c_float()
        _lib.check(self._lib.dpcn_train_step_device(
            self._h, ctypes.c_void_p(xp), xn, ctypes.c_void_p(yp), yn, int(inference_steps),
            ctypes.byref(e) if read_energy else None))
        return float(e.value) if read_energy else None

    def predict(self, X, inference_steps: Optional[int] = None, with_projection: bool = True):
        self._require_configured()
        steps = self.default_inference_steps if inference_steps is None else inference_steps
        x = _f32(X)
        out = np.empty(self.batch_size * self.terminal_size, dtype=np.float32)
        _lib.check(self._lib.dpcn_predict(self._h, _ptr(x), x.size, int(steps),
                                          int(with_projection), _ptr(out), out.size))
        return out.reshape(self.batch_size, self.terminal_size)

    def fit(self, X, Y, epochs: int, inference_steps: int = 1, initial_lr: Optional[float] = None,
            decay_rate: float = 1.0, shuffle: bool = True, verbose: bool = False,
            device_resident: bool = True):
        """Epoch loop of ``deepity/utils.py:19-143`` without the progress bars.

        ``device_resident`` (default): the data set is uploaded once, every epoch's permutation
        (``np.random.permutation``, as in the reference, so a seeded run visits the same batches)
        goes up as an index vector, and each mini-batch is gathered on the device straight into the
        step's inputs -- no host slicing, no per-batch upload, no host synchronisation except one
        energy read per epoch (every step when ``verbose``).  ``device_resident=False`` slices on
        the host and calls ``train_step`` per batch."""
        self._require_configured()
        X = np.ascontiguousarray(X, dtype=np.float32)
        Y = np.ascontiguousarray(Y, dtype=np.float32)
        n, bsz = len(X), self.batch_size
        if n == 0:
            raise ValueError("Training data cannot be empty.")
        if n % bsz != 0:
            raise ValueError(f"Number of samples ({n}) must be divisible by batch_size ({bsz}).")
        if initial_lr is None:
            initial_lr = self._learning_rate
        batches = n // bsz
        if not device_resident:
            for epoch in range(epochs):
                self.set_learning_rate(initial_lr * (decay_rate ** epoch))
                idx = np.random.permutation(n) if shuffle else np.arange(n)
                total = 0.0
                for b in range(batches):
                    sel = idx[b * bsz:(b + 1) * bsz]
                    total += self.train_step(X[sel], Y[sel], inference_steps)
                if verbose:
                    print(f"epoch {epoch + 1} avg energy = {total / batches:.4f}")
            return self

        import torch
        lib = self._lib
        ctx = lib.dpcn_context(self._h)
        device = torch.device("cuda", self._device_index)
        stream = torch.cuda.ExternalStream(lib.dpc_stream(ctx), device=device)
        X2, Y2 = X.reshape(n, -1), Y.reshape(n, -1)
        with torch.cuda.stream(stream):
            Xd = torch.from_numpy(X2).to(device)
            Yd = torch.from_numpy(Y2).to(device)
            xb = torch.empty((bsz, X2.shape[1]), dtype=torch.float32, device=device)
            yb = torch.empty((bsz, Y2.shape[1]), dtype=torch.float32, device=device)
            for epoch in range(epochs):
                self.set_learning_rate(initial_lr * (decay_rate ** epoch))
                idx = np.random.permutation(n) if shuffle else np.arange(n)
                order = torch.from_numpy(np.ascontiguousarray(idx, dtype=np.int64)).to(device)
                total = 0.0
                for b in range(batches):
                    for src, dst in ((Xd, xb), (Yd, yb)):
                        _lib.check(lib.dpc_gather_rows(
                            ctx, ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(order.data_ptr()),
                            b * bsz, bsz, src.shape[1], ctypes.c_void_p(dst.data_ptr())))
                    read = verbose or b == batches - 1
                    energy = self.train_step_device(xb, yb, inference_steps, read_energy=read)
                    if verbose:
                        total += energy
                if verbose:
                    print(f"epoch {epoch + 1} avg energy = {total / batches:.4f}")
            stream.synchronize()
        return self

    def set_gradient_sync(self, reduce_fn, global_batch: int) -> None:
        """Batch sharding: this network holds ``batch_size`` of ``global_batch`` rows.
        ``reduce_fn(t)`` gets a CUDA torch view of the staged gradient sums and must sum it in
        place over all shards (``torch.distributed.all_reduce``); it runs with the library's
        stream current.  ``None`` switches back to the fused single-process updates."""
        self._require_configured()
        if reduce_fn is None:
            _lib.check(self._lib.dpcn_set_gradient_sync(self._h, None, None, 0))
            self._sync_cb = None
            return
        import torch
        lib = self._lib
        device = torch.device("cuda", self._device_index)

        def trampoline(user, dev, count, stream):
            try:
                class _View:
                    __cuda_array_interface__ = {"shape": (int(count),), "typestr": "<f4",
                                                "data": (int(dev), False), "version": 3}
                t = torch.as_tensor(_View(), device=device)
                with torch.cuda.stream(torch.cuda.ExternalStream(int(stream), device=device)):
                    reduce_fn(t)
                return 0
            except Exception as exc:  # noqa: BLE001 - reported through the status code
                self._sync_error = exc
                return 1

        proto = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                 ctypes.c_void_p)
        self._sync_cb = proto(trampoline)  # keep the thunk alive as long as it is installed
        _lib.check(lib.dpcn_set_gradient_sync(self._h, ctypes.cast(self._sync_cb, ctypes.c_void_p),
                                              None, int(global_batch)))

    # -- checkpoint surface: the reference's tensor names (docs/model-format.md:104-117) ------
    _PUBLIC = {"W": "weight", "b": "bias", "Psi": "psi"}

    def _state_entries(self):
        lib, out = self._lib, []
        layer, rows, cols, stride, opt = (ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64(),
                                          ctypes.c_int64(), ctypes.c_int())
        name = ctypes.create_string_buffer(32)
        for i in range(_lib.check(lib.dpcn_state_dict_size(self._h))):
            _lib.check(lib.dpcn_state_dict_entry(self._h, i, ctypes.byref(layer), name, 32,
                                                 ctypes.byref(rows), ctypes.byref(cols),
                                                 ctypes.byref(stride), ctypes.byref(opt)))
            out.append((layer.value, name.value.decode(), rows.value, cols.value, bool(opt.value)))
        return out

    def state_dict(self) -> dict:
        """``layers.{i}.weight|bias|psi`` -> numpy array, the names and shapes the reference's
        ``save()`` writes (``Layer::GetStateDict``)."""
        self._require_configured()
        out = {}
        for layer, name, rows, cols, opt in self._state_entries():
            if not opt:
                a = self.get_tensor(layer, name)
                out[f"layers.{layer}.{self._PUBLIC[name]}"] = a.reshape(cols) if rows == 1 \
                    else a.reshape(rows, cols)
        return out

    def optimizer_state_dict(self) -> dict:
        """``optimizer.layers.{i}.{weight,bias,psi}.{m,v}`` plus the step counters
        ``optimizer.layers.{i}.step`` / ``psi_step`` (int32, shape [1]): what the reference's
        ``save_checkpoint`` adds to the weights (``Layer::GetOptimizerStateDict`` and
        ``GetOptimizerCounters``)."""
        self._require_configured()
        out, layers = {}, set()
        for layer, name, rows, cols, opt in self._state_entries():
            layers.add(layer)
            if opt:
                a = self.get_tensor(layer, name)
                out[f"optimizer.layers.{layer}.{name}"] = a.reshape(cols) if rows == 1 \
                    else a.reshape(rows, cols)
        for layer in sorted(layers):
            for counter in ("step", "psi_step"):
                v = ctypes.c_int32()
                if self._lib.dpcn_get_counter(self._h, layer, counter.encode(), ctypes.byref(v)) == 0:
                    out[f"optimizer.layers.{layer}.{counter}"] = np.asarray([v.value], dtype=np.int32)
        return out

    def load_state_dict(self, state: dict, strict: bool = True) -> None:
        """Inverse of ``state_dict()`` + ``optimizer_state_dict()`` (either or both merged into
        one mapping).  ``strict``: every tensor this network owns must be present."""
        self._require_configured()
        back = {v: k for k, v in self._PUBLIC.items()}
        seen = set()
        for key, value in state.items():
            parts = key.split(".")
            if parts[0] == "optimizer":
                layer, name = int(parts[2]), ".".join(parts[3:])
                if name in ("step", "psi_step"):
                    _lib.check(self._lib.dpcn_set_counter(self._h, layer, name.encode(),
                                                          int(np.asarray(value).ravel()[0])))
                    continue
            else:
                layer, name = int(parts[1]), back[parts[2]]
            self.set_tensor(layer, name, value)
            seen.add((layer, name))
        if strict:
            missing = [f"{l}.{n}" for l, n, _, _, _ in self._state_entries() if (l, n) not in seen]
            if missing:
                raise KeyError(f"load_state_dict: missing tensors {missing[:6]}")

    @property
    def launch_count(self) -> int:
        return int(self._lib.dpcn_launch_count(self._h))

    def train_step_flops(self, inference_steps: int) -> float:
        return float(self._lib.dpcn_train_step_flops(self._h, int(inference_steps)))


class DKPPCN(_Network):
    """Predictive-coding network with Direct Kolen-Pollack feedback (deepity/DKPPCN.py)."""
    KIND, NAME = KIND_DKP, "DKPPCN"

    def configure(self, learning_rate: float = 1e-6, inference_rate: float = 0.1,
                  feedback_rate: float = 1e-4, lmbda: float = 1e-2, optimizer: str = "SGD",
                  psi_optimizer: str = "SGD", center_weights: bool = False,
                  psi_decay: Optional[float] = None, seed: Optional[int] = None,
                  precision: str = "fp32") -> "DKPPCN":
        self._learning_rate, self._inference_rate = learning_rate, inference_rate
        self._feedback_rate, self._lambda = feedback_rate, lmbda
        self._build_backend(learning_rate, inference_rate, feedback_rate, lmbda)
        self.set_optimizer(optimizer)
        self.set_psi_optimizer(psi_optimizer)
        self.set_precision(precision)
        _lib.check(self._lib.dpcn_compile(self._h))
        self._configured = True
        self.randomize_weights(seed)
        self.set_center_weights(center_weights)
        self.set_psi_decay(-1.0 if psi_decay is None else psi_decay)
        return self

    def set_psi_optimizer(self, optimizer: str) -> None:
        self._option("psi_optimizer", OPT_IDS[optimizer.upper()])
        self._psi_optimizer = optimizer

    def set_psi_decay(self, decay: float) -> None:
        self._option("psi_decay", 0, decay)

    def set_feedback_rate(self, feedback_rate: float) -> None:
        self._option("feedback_rate", 0, feedback_rate)
        self._feedback_rate = feedback_rate


class FullPCN(DKPPCN):
    """DKP + muPC scaling, residuals, iPC, momentum, softmax-CE head (deepity/FullPCN.py)."""
    KIND, NAME = KIND_FULL, "FullPCN"

    def configure(self, learning_rate: float = 1e-6, inference_rate: float = 0.1,
                  feedback_rate: float = 1e-4, lmbda: float = 1e-2, optimizer: str = "SGD",
                  psi_optimizer: str = "SGD", use_mu_pc_scaling: bool = False,
                  use_residual_connections: bool = False, use_ipc: bool = False,
                  use_epc: bool = False, use_momentum: bool = False, momentum_beta: float = 0.9,
                  use_cross_entropy: bool = False, seed: Optional[int] = None,
                  dist: str = "normal", center_weights: bool = False,
                  precision: str = "fp32") -> "FullPCN":
        self._learning_rate, self._inference_rate = learning_rate, inference_rate
        self._feedback_rate, self._lambda = feedback_rate, lmbda
        self._build_backend(learning_rate, inference_rate, feedback_rate, lmbda)
        self._option("mupc", int(use_mu_pc_scaling))
        self._option("residual", int(use_residual_connections))
        self._option("ipc", int(use_ipc))
        self._option("epc", int(use_epc))
        self._option("momentum", int(use_momentum), momentum_beta)
        self._option("cross_entropy", int(use_cross_entropy))
        self.set_optimizer(optimizer)
        self.set_psi_optimizer(psi_optimizer)
        self.set_precision(precision)
        _lib.check(self._lib.dpcn_compile(self._h))
        self._configured = True
        self.randomize_weights(seed)
        self.set_center_weights(center_weights)
        return self


class SimplePCN(_Network):
    """Classic predictive coding, mu = W f(z) + b (deepity/SimplePCN.py)."""
    KIND, NAME = KIND_SIMPLE, "SimplePCN"

    def configure(self, learning_rate: float = 1e-4, inference_rate: float = 1e-4,
                  lmbda: float = 0.0001, optimizer: str = "SGD", seed: Optional[int] = None,
                  dist: str = "normal", center_weights: bool = False,
                  use_cross_entropy: bool = False, precision: str = "fp32") -> "SimplePCN":
        self._learning_rate, self._inference_rate, self._lambda = learning_rate, inference_rate, lmbda
        self._build_backend(learning_rate, inference_rate, 0.0, lmbda)
        self._option("cross_entropy", int(use_cross_entropy))
        self.set_optimizer(optimizer)
        self.set_precision(precision)
        _lib.check(self._lib.dpcn_compile(self._h))
        self._configured = True
        self.randomize_weights(seed)
        self.set_center_weights(center_weights)
        return self

    def train_step(self, X, Y, steps: int = 1) -> float:
        """The reference's Python-level loop (deepity/SimplePCN.py:269-293): settle ``steps``
        times, summing the energy of every step, then update the weights."""
        return self._train(2, X, Y, steps)

    def train_step_native(self, X, Y, steps: int) -> float:
        """SimplePCNetwork::TrainStep (final energy only)."""
        return self._train(0, X, Y, steps)

    def train_step_with_projection(self, X, Y, steps: int) -> float:
        """SimplePCNetwork::TrainStepWithProjection."""
        return self._train(1, X, Y, steps)

    def predict(self, X, inference_steps: Optional[int] = None, with_projection: bool = False):
        return super().predict(X, inference_steps, with_projection)

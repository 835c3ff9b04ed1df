"""Layer-sharded DKPPCN across the GPUs of one node.

Deep stacks are split into contiguous blocks of layers, one block per rank (one process per
GPU).  Every phase of the train step except the forward sweep is local to a layer and its
two neighbours, so a rank only ever exchanges ONE boundary tensor with the rank above or
below it per phase, plus a broadcast of the small terminal error:

    forward sweep   rank r sends the prediction of its top layer to r+1          [B, H]
    terminal error  last rank broadcasts e_T (after the sweep and after the last
                    settling pass, which is the one the Psi update reads)         [B, TS]
    settling pass   a) every rank computes errors/predictions of its block, then
                       sends the error of the boundary layer UP (the rank above
                       owns that layer's belief and needs e to update it)        [B, H]
                    b) every rank updates its beliefs, then sends the boundary
                       belief DOWN (the rank below needs it for its next error)  [B, H]
    learn           the rank above sends Psi of its first layer DOWN once per step
                    (the direct-feedback update of the layer below reads it)     [H, TS]
    energy          one all-reduce of a scalar

The local block of a rank is an ordinary network of this library whose last layer is a
"ghost": a copy of the first layer of the rank above (its belief z, error e and Psi), so the
single-GPU kernels run unchanged on it.  The reference has no multi-GPU code at all; the
arithmetic per layer is exactly that of the single-GPU path, so results are identical to it
up to the order of the energy sum.

The schedule is written against a small engine interface so that the same code is tested on
CPU ranks (gloo) with an engine backed by the numpy oracle (tests/test_sharded_cpu.py).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Sequence, Tuple

import numpy as np


def partition_layers(n_weight_layers: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) ranges of weight layers per rank, sizes differing by at most 1;
    the remainder goes to the lowest ranks.  Every rank gets at least one layer."""
    if world < 1 or n_weight_layers < world:
        raise ValueError(f"cannot split {n_weight_layers} weight layers over {world} ranks")
    base, rem = divmod(n_weight_layers, world)
    out, b = [], 0
    for r in range(world):
        e = b + base + (1 if r < rem else 0)
        out.append((b, e))
        b = e
    return out


class GpuEngine:
    """The local block on one GPU, driven phase by phase through the dpc_* C ABI."""

    def __init__(self, sizes: Sequence[int], batch: int, hyper: dict, act: str, ghost_top: bool,
                 terminal_size: int, device: int, precision: str = "fp32"):
        import torch
        from . import _lib
        from .layer import ACT_IDS
        self.torch = torch
        self.lib = _lib.load()
        self.check = _lib.check
        self.batch, self.sizes, self.ts = batch, list(sizes), terminal_size
        self.n = len(self.sizes)  # local layers incl. ghost / terminal
        self.h = ctypes.c_void_p()
        self.check(self.lib.dpcn_create(1, batch, device, ctypes.byref(self.h)))
        for i in range(self.n - 1):
            self.check(self.lib.dpcn_add_layer(self.h, self.sizes[i], self.sizes[i + 1],
                                               terminal_size, hyper["lr"], hyper["ir"],
                                               hyper["fl"], hyper["lmbda"], ACT_IDS[act]))
        self.check(self.lib.dpcn_add_layer(self.h, self.sizes[-1], 0, terminal_size, hyper["lr"],
                                           hyper["ir"], hyper["fl"], hyper["lmbda"],
                                           ACT_IDS["linear"]))
        self.check(self.lib.dpcn_set_option(self.h, b"ghost_top", int(ghost_top), 0.0))
        self.check(self.lib.dpcn_set_option(self.h, b"precision", {"fp32": 0, "tf32": 1, "mixed": 2}[precision],
                                            0.0))
        self.check(self.lib.dpcn_compile(self.h))
        self.ctx = self.lib.dpcn_context(self.h)
        self.plan = self.lib.dpcn_plan(self.h)
        self.stream = torch.cuda.ExternalStream(self.lib.dpc_stream(self.ctx),
                                                device=torch.device("cuda", device))
        self.ghost_top = ghost_top
        self._views = {}
        # activations whose derivative is a function of their output (see dpc_direct_feedback)
        self.output_deriv = act in ("tanh", "sigmoid", "relu", "linear", "hard_tanh")

    # -- tensors as torch views over the library's device memory (zero copy) ---------------
    def tensor(self, layer: int, name: str):
        key = (layer, name)
        if key not in self._views:
            p = ctypes.c_void_p()
            stride = ctypes.c_int64()
            n = self.lib.dpcn_tensor_size(self.h, layer, name.encode())
            self.check(self.lib.dpcn_tensor_ptr(self.h, layer, name.encode(), ctypes.byref(p),
                                                ctypes.byref(stride)))

            class _View:
                __cuda_array_interface__ = {"shape": (int(n),), "typestr": "<f4",
                                            "data": (int(p.value), False), "version": 3}
            self._views[key] = self.torch.as_tensor(_View(), device=self.stream.device)
        return self._views[key]

    def set_param(self, layer: int, name: str, value) -> None:
        v = np.ascontiguousarray(value, dtype=np.float32).ravel()
        from . import _lib
        self.check(self.lib.dpcn_set_tensor(self.h, layer, name.encode(),
                                            v.ctypes.data_as(_lib.c_f32p), v.size))

    def get(self, layer: int, name: str) -> np.ndarray:
        self.sync()
        return self.tensor(layer, name).cpu().numpy()

    def terminal_error_tensor(self):
        return self.tensor(self.n - 1, "eT" if self.ghost_top else "e")

    # -- phases ---------------------------------------------------------------------------
    def reset(self):
        self.check(self.lib.dpcn_reset_state(self.h))

    def project_forward(self, skip_last_copy: bool):
        # Inside a train step nothing reads mu / preact of the swept layers before they are
        # recomputed (the direct-feedback update takes f' from the copied outputs), so the sweep
        # only writes the beliefs of the layers above.
        extra = (512 | 2048) if self.output_deriv else 0  # DPC_FWD_NO_MU | DPC_FWD_NO_PREACT
        self.check(self.lib.dpc_project_forward_ex(self.plan, 0, self.n - 1, int(skip_last_copy),
                                                   extra))

    def terminal_error(self):
        self.check(self.lib.dpc_error(self.plan, self.n - 1, 0))

    def dfa(self):
        # 2 = DPC_DFA_FROM_OUTPUT: z[l+1] still equals f(preact[l]) right after the sweep
        self.check(self.lib.dpc_direct_feedback(self.plan, 0, self.n - 1,
                                                2 if self.output_deriv else 0))

    def forward_state(self, first_cached: bool, flags: int):
        """ComputeMuOnly + error of the layer above for every local weight layer."""
        start = 0
        if first_cached:
            self.check(self.lib.dpc_forward(self.plan, 0, 1, (flags | 16) & ~256))  # CACHED
            start = 1
        if self.n - 1 - start > 0:
            self.check(self.lib.dpc_forward(self.plan, start, self.n - 1 - start, flags))

    def update_state(self, first: int, count: int):
        if count > 0:
            self.check(self.lib.dpc_update_state(self.plan, first, count))

    def update_weights(self):
        self.check(self.lib.dpc_update_weights(self.plan, 0, self.n - 1, 0))

    def energy_reset(self):
        self.check(self.lib.dpc_energy_reset(self.plan))

    def energy_read(self) -> float:
        e = ctypes.c_double()
        self.check(self.lib.dpc_energy_read(self.plan, ctypes.byref(e)))
        return e.value

    def sync(self):
        self.check(self.lib.dpc_sync(self.ctx))

    def mark_clamped(self, layer: int):
        """The kernels take clamping from the ranges the schedule passes; nothing to record."""

    def wrote_belief(self, layer: int):
        """The schedule wrote z of `layer` itself (a copy or an NCCL receive into the library's
        memory): the tensor-core kernels' operand copies of it must be rebuilt."""
        self.check(self.lib.dpc_plan_invalidate(self.plan, layer, 1, 1))  # DPC_WROTE_Z

    def close(self):
        """Free the block's device memory (the network, its plan and context, its stream).
        Every torch tensor that was used on the block's stream must have been released before:
        torch's allocator records an event on each stream a tensor was used on when the tensor is
        freed, and aborts the process if that stream no longer exists."""
        if self.h:
            self.torch.cuda.synchronize()
            self._views.clear()
            self.lib.dpcn_destroy(self.h)
            self.h = None

    def comm_stream(self):
        return self.torch.cuda.stream(self.stream)

    @property
    def launch_count(self) -> int:
        return int(self.lib.dpc_launch_count(self.ctx))


FWD_COPY, FWD_ERR, FWD_ENERGY, FWD_FE, FWD_TRANSIENT = 1, 2, 4, 8, 256


class ShardedDKPPCN:
    """DKPPCN whose weight layers are split over the ranks of a torch.distributed group."""

    def __init__(self, sizes: Sequence[int], batch: int, hyper: dict, act: str = "tanh",
                 engine_factory=None, group=None, precision: str = "fp32"):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.sizes, self.batch = list(sizes), batch
        self.ts = self.sizes[-1]
        n_weight = len(self.sizes) - 1
        self.ranges = partition_layers(n_weight, self.world)
        self.begin, self.end = self.ranges[self.rank]
        self.is_first, self.is_last = self.rank == 0, self.rank == self.world - 1
        # local widths: own layers' inputs + the input width of the layer above (ghost), or the
        # real terminal on the last rank
        local = self.sizes[self.begin:self.end + 1]
        if engine_factory is None:
            device = int(os.environ.get("LOCAL_RANK", self.rank))
            engine_factory = lambda **kw: GpuEngine(device=device, precision=precision, **kw)  # noqa: E731
        self.eng = engine_factory(sizes=local, batch=batch, hyper=hyper, act=act,
                                  ghost_top=not self.is_last, terminal_size=self.ts)
        self.n = len(local)

    # ---- parameter placement: global layer index -> local ---------------------------------
    def owns(self, layer: int) -> bool:
        return self.begin <= layer < self.end

    def set_param(self, layer: int, name: str, value) -> None:
        if self.owns(layer):
            self.eng.set_param(layer - self.begin, name, value)

    def get_local(self, layer: int, name: str):
        return self.eng.get(layer - self.begin, name)

    # ---- checkpoint surface: global tensor names, one shard per rank ------------------------
    def local_state_dict(self) -> dict:
        """This rank's parameters under the names a single-process network gives them
        (``layers.{global index}.weight|bias|psi``, docs/model-format.md:104-117 of the
        reference): the shard a per-rank checkpoint file holds."""
        out = {}
        for g in range(self.begin, self.end):
            s, n = self.sizes[g], self.sizes[g + 1]
            out[f"layers.{g}.weight"] = np.asarray(self.get_local(g, "W")).reshape(n, s)
            out[f"layers.{g}.bias"] = np.asarray(self.get_local(g, "b")).reshape(n)
            out[f"layers.{g}.psi"] = np.asarray(self.get_local(g, "Psi")).reshape(s, self.ts)
        return out

    def gather_state_dict(self, dst: int = 0):
        """The whole network's state dict on rank ``dst`` (None elsewhere)."""
        parts = [None] * self.world if self.rank == dst else None
        self.dist.gather_object(self.local_state_dict(), parts, dst=dst, group=self.group)
        if parts is None:
            return None
        merged = {}
        for part in parts:
            merged.update(part)
        return merged

    def load_state_dict(self, state: dict) -> None:
        """Takes the tensors of the layers this rank owns from a whole-network (or per-rank)
        state dict; names of other ranks' layers are ignored."""
        names = {"weight": "W", "bias": "b", "psi": "Psi"}
        for key, value in state.items():
            _, index, kind = key.split(".")
            if self.owns(int(index)):
                self.set_param(int(index), names[kind], value)

    # ---- communication helpers -------------------------------------------------------------
    def _exchange(self, send=None, recv=None):
        """send/recv: (tensor, peer rank) or None.  A send and a receive of the same phase go
        out as ONE batched point-to-point group (a single NCCL group call: neither waits for
        the other, and the backend does not serialise them)."""
        ops = []
        if send is not None:
            ops.append(self.dist.P2POp(self.dist.isend, send[0], send[1], group=self.group))
        if recv is not None:
            ops.append(self.dist.P2POp(self.dist.irecv, recv[0], recv[1], group=self.group))
        if not ops:
            return
        with self.eng.comm_stream():
            for work in self.dist.batch_isend_irecv(ops):
                work.wait()

    def _broadcast_terminal_error(self):
        with self.eng.comm_stream():
            self.dist.broadcast(self.eng.terminal_error_tensor(), self.world - 1, group=self.group)

    # ---- one train step ---------------------------------------------------------------------
    def train_step(self, x, y, steps: int, read_energy: bool = True):
        eng, n = self.eng, self.n
        up, down = self.rank + 1, self.rank - 1
        eng.reset()
        if self.is_first:
            self._load(0, "z", x)
            eng.mark_clamped(0)
        if self.is_last:
            self._load(n - 1, "z", y)
            eng.mark_clamped(n - 1)
        # Psi of the first layer of the rank above, for this step's direct-feedback update.
        if self.world > 1:
            self._exchange(send=None if self.is_first else (eng.tensor(0, "Psi"), down),
                           recv=None if self.is_last else (eng.tensor(n - 1, "Psi"), up))
        # forward sweep, rank after rank
        if not self.is_first:
            self._exchange(recv=(eng.tensor(0, "z"), down))
            eng.wrote_belief(0)
        eng.project_forward(skip_last_copy=self.is_last)
        if not self.is_last:
            self._exchange(send=(eng.tensor(n - 1, "z"), up))
        if self.is_last:
            eng.terminal_error()
        if self.world > 1:
            self._broadcast_terminal_error()
        eng.dfa()
        first_unclamped = 1 if self.is_first else 0
        for t in range(steps):
            eng.forward_state(self.is_first, FWD_ERR | FWD_FE | FWD_TRANSIENT)
            if self.world > 1:
                self._exchange(send=None if self.is_last else (eng.tensor(n - 1, "e"), up),
                               recv=None if self.is_first else (eng.tensor(0, "e"), down))
                if t == steps - 1:
                    self._broadcast_terminal_error()
            eng.update_state(first_unclamped, n - 1 - first_unclamped)
            if self.world > 1:
                self._exchange(send=None if self.is_first else (eng.tensor(0, "z"), down),
                               recv=None if self.is_last else (eng.tensor(n - 1, "z"), up))
        eng.forward_state(self.is_first, FWD_FE | FWD_TRANSIENT)
        eng.update_weights()
        eng.energy_reset()
        # last pass: errors and energy only (nobody reads fe or the predictions afterwards)
        eng.forward_state(self.is_first, FWD_ERR | FWD_ENERGY | FWD_TRANSIENT)
        if self.world > 1:
            # leave the boundary error where a reader of the rank above expects it
            self._exchange(send=None if self.is_last else (eng.tensor(n - 1, "e"), up),
                           recv=None if self.is_first else (eng.tensor(0, "e"), down))
        if not read_energy:
            return None
        energy = eng.energy_read()
        if self.world > 1:
            import torch
            t = torch.tensor([energy], dtype=torch.float64)
            if self.dist.get_backend(self.group) == "nccl":
                t = t.cuda()
            self.dist.all_reduce(t, group=self.group)
            energy = float(t.item())
        return energy

    def _load(self, layer: int, name: str, value):
        import torch
        t = self.eng.tensor(layer, name)
        src = value if isinstance(value, torch.Tensor) else torch.from_numpy(
            np.ascontiguousarray(value, dtype=np.float32))
        with self.eng.comm_stream():
            t.copy_(src.reshape(-1).to(t.device, non_blocking=True))
        if name == "z":
            self.eng.wrote_belief(layer)

    def close(self):
        if hasattr(self.eng, "close"):
            self.eng.close()

    def train_step_flops(self, steps: int) -> float:
        from .flops import algorithmic_flops
        return algorithmic_flops("dkp", self.sizes, self.batch, steps)


# ------------------------------------------------------------------------------------------
class BatchSharded:
    """Wide, shallow networks split over the ranks by batch rows.

    Every rank holds the full W, b, Psi (and optimizer moments) and ``global_batch / world``
    rows of every belief, error and prediction.  Settling, the softmax head and momentum are
    row-local and need no communication; only the weight-shaped sums couple rows:

        direct-feedback update   one all-reduce of the staged  proj^T z  of all layers
        learn                    one all-reduce of the staged  fe^T z, column sums of fe and
                                 z^T e_T  of all layers (a single contiguous buffer)
        energy                   one all-reduce of a scalar

    The sums are raw (no 1/B, no learning rate), so SGD, Adam and AdamW all apply them with
    the global batch exactly as a single process would; iPC mode all-reduces in every
    settling step because it learns in every step.  ``build_local(local_batch)`` returns the
    rank's network: a configured deepity_b200 network, or anything with the same
    ``set_gradient_sync(reduce_fn, global_batch)`` / ``train_step`` pair (the CPU tests use
    the numpy oracle).  Parameters must be set identically on every rank.
    """

    def __init__(self, build_local, global_batch: int, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if global_batch % self.world != 0:
            raise ValueError(f"global batch {global_batch} does not split over {self.world} ranks")
        self.global_batch, self.local_batch = global_batch, global_batch // self.world
        self.net = build_local(self.local_batch)
        self.net.set_gradient_sync(self._reduce, global_batch)

    def _reduce(self, t):
        if self.world > 1:
            self.dist.all_reduce(t, group=self.group)

    def rows(self, a):
        """This rank's rows of a [global_batch, ...] array."""
        return a[self.rank * self.local_batch:(self.rank + 1) * self.local_batch]

    def _energy(self, local):
        import torch
        if self.world == 1 or local is None:
            return local
        t = torch.tensor([local], dtype=torch.float64)
        if self.dist.get_backend(self.group) == "nccl":
            t = t.cuda()
        self.dist.all_reduce(t, group=self.group)
        return float(t.item())

    def train_step(self, X, Y, inference_steps: int = 1) -> float:
        """X, Y: the GLOBAL batch on the host; every rank takes its rows."""
        return self._energy(self.net.train_step(self.rows(X), self.rows(Y), inference_steps))

    def train_step_device(self, x_local, y_local, inference_steps: int = 1, read_energy=True):
        """x_local, y_local: this rank's rows, already on its GPU."""
        return self._energy(self.net.train_step_device(x_local, y_local, inference_steps,
                                                       read_energy))

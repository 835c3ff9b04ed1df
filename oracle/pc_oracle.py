"""numpy restatement of the reference's CPU predictive-coding train step.

TEST INFRASTRUCTURE ONLY: the product never imports this module.  It exists so
that parity tests and the benchmark's CPU leg have an oracle that does not depend
on the reference checkout being present.  Every function cites the reference
file:line it follows.  Parity pin: ``tests/test_oracle_pin.py`` checks this
module against the compiled reference (``oracle/_ref``) when that library exists
and against the fixtures under ``tests/golden/`` (generated from the compiled
reference by ``tests/golden/make_golden.py``) always.

All arithmetic is float32 like the reference's ``float`` backend; GEMMs go to
numpy's BLAS, transcendental functions to numpy (the reference uses SLEEF u10 /
libm: agreement is to a few ulp, parity is judged at 1e-4 relative).
"""
from __future__ import annotations

import numpy as np

F = np.float32

GELU_1 = F(0.7978845608)  # sqrt(2/pi)       include/deepity/utils/activations/Gelu.h:19-22
GELU_2 = F(0.044715)


def act(name: str, z: np.ndarray) -> np.ndarray:
    """Forward activation, include/deepity/utils/Activations.h:44-72."""
    z = z.astype(F, copy=False)
    if name == "relu":
        return np.where(z > 0, z, F(0)).astype(F)
    if name == "gelu":
        inner = GELU_1 * z + (GELU_2 * GELU_1) * (z * z) * z
        return (F(0.5) * z * (F(1) + np.tanh(inner))).astype(F)
    if name == "sigmoid":
        return (F(1) / (F(1) + np.exp(-z))).astype(F)
    if name == "esigmoid":
        return (F(0.5) + F(0.5) * (z / (F(1) + np.abs(z)))).astype(F)
    if name == "tanh":
        return np.tanh(z).astype(F)
    if name == "hard_tanh":
        return np.clip(z, F(-1), F(1)).astype(F)
    return z


def dact(name: str, z: np.ndarray) -> np.ndarray:
    """Derivative from the pre-activation, include/deepity/utils/Activations.h:79-115."""
    z = z.astype(F, copy=False)
    if name == "relu":
        return (z > 0).astype(F)
    if name == "gelu":
        zsq = z * z
        inner = GELU_1 * z + (GELU_2 * GELU_1) * zsq * z
        t = np.tanh(inner)
        gp = GELU_1 + (F(3) * GELU_2 * GELU_1) * zsq
        return (F(0.5) * (F(1) + t) + F(0.5) * z * gp * (F(1) - t * t)).astype(F)
    if name == "sigmoid":
        s = F(1) / (F(1) + np.exp(-z))
        return (s * (F(1) - s)).astype(F)
    if name == "esigmoid":
        a = F(1) + np.abs(z)
        return (F(0.5) / (a * a)).astype(F)
    if name == "tanh":
        t = np.tanh(z)
        return (F(1) - t * t).astype(F)
    if name == "hard_tanh":
        return ((z > -1) & (z < 1)).astype(F)
    return np.ones_like(z, dtype=F)


def softmax_ce(z, mu):
    """e = z - softmax(mu), E = -sum z*log(p+1e-8); src/backend/CPUBackend.cpp:658-695."""
    m = mu.max(axis=1, keepdims=True)
    ex = np.exp((mu - m).astype(F)).astype(F)
    p = (ex / ex.sum(axis=1, keepdims=True, dtype=F)).astype(F)
    energy = F(-(z * np.log(p + F(1e-8))).sum(dtype=F))
    return (z - p).astype(F), float(energy)


def adam_step(p, g, m, v, t, lr, b1=F(0.9), b2=F(0.999), eps=F(1e-8), wd=None):
    """src/backend/CPUBackend.cpp:721-772 with the chunk kernels of
    src/backend/CPUBackendHighway.cpp:779-840.  ``wd`` = lr*weightDecay (AdamW)."""
    b1t = F(1) - F(b1) ** F(t)
    b2t = F(1) - F(b2) ** F(t)
    step = F(lr) * np.sqrt(b2t, dtype=F) / b1t
    m[...] = b1 * m + (F(1) - b1) * g
    v[...] = b2 * v + (F(1) - b2) * (g * g)
    if wd is not None:
        p -= F(wd) * p
    p -= step * m / (np.sqrt(v) + eps)


def center_rows(W):
    """src/backend/CPUBackend.cpp:250-272."""
    W -= (W.sum(axis=1, keepdims=True, dtype=F) / F(W.shape[1])).astype(F)


class _Layer:
    def __init__(self, s, n, ts, B, lr, ir, fl, lmbda, act_name):
        self.s, self.n, self.ts, self.B = s, n, ts, B
        self.lr, self.ir, self.fl, self.lmbda, self.act = F(lr), F(ir), F(fl), F(lmbda), act_name
        self.z = np.zeros((B, s), F)
        self.e = np.zeros((B, s), F)
        self.clamped = False
        self.cache_valid = False
        self.a = F(1)
        self.residual = False
        self.cross_entropy = False
        self.momentum = None
        self.v = None
        if n > 0:
            self.W = np.zeros((n, s), F)
            self.b = np.zeros(n, F)
            self.mu = np.zeros((B, n), F)
            self.preact = np.zeros((B, n), F)
            self.cmu = np.zeros((B, n), F)
            self.cpre = np.zeros((B, n), F)
            self.Psi = np.zeros((s, ts), F)
            self.adj = np.zeros((B, s), F)
            self.mW, self.vW = np.zeros((n, s), F), np.zeros((n, s), F)
            self.mb, self.vb = np.zeros(n, F), np.zeros(n, F)
            self.mP, self.vP = np.zeros((s, ts), F), np.zeros((s, ts), F)
            self.t = 0
            self.tP = 0


class PCOracle:
    """DirectKP ('dkp'), Full ('full') and Simple ('simple') networks, CPU semantics."""

    def __init__(self, kind, sizes, batch, *, lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh",
                 last_act=None, optimizer="SGD", psi_optimizer="SGD", psi_decay=-1.0,
                 center_weights=False, cross_entropy=False, mupc=False, residual=False,
                 ipc=False, epc=False, momentum=None, terminal_size=None):
        self.kind, self.B, self.sizes = kind, batch, list(sizes)
        # terminal_size differs from sizes[-1] only for one block of a layer-sharded network,
        # whose last layer is a copy of the next block's first layer (tests/test_sharded_cpu.py).
        ts = self.sizes[-1] if terminal_size is None else terminal_size
        self.e_terminal = None  # override of the terminal error for such a block
        # Batch sharding: grad_sync(phase, layer, [arrays]) returns the arrays summed over the
        # shards, global_B the batch those sums cover (no counterpart in the reference).
        self.grad_sync = None
        self.global_B = None
        nw = len(self.sizes) - 1
        self.layers = []
        for i in range(nw):
            a = act if (i + 1 < nw or last_act is None) else last_act
            self.layers.append(_Layer(self.sizes[i], self.sizes[i + 1], ts, batch, lr, ir, fl,
                                      lmbda, a))
        self.layers.append(_Layer(self.sizes[-1], 0, ts, batch, lr, ir, fl, lmbda, "linear"))
        self.opt, self.opt_psi = optimizer, psi_optimizer
        self.psi_decay, self.center = F(psi_decay), center_weights
        self.ipc, self.epc = ipc, epc
        self.layers[-1].cross_entropy = cross_entropy
        if momentum is not None:
            for l in self.layers:
                l.momentum = F(momentum)
                l.v = np.zeros((batch, l.s), F)
        if kind == "full":
            self._wire_mupc(mupc, residual)

    # src/networks/FullPCNetwork.cpp:405-465
    def _wire_mupc(self, mupc, residual):
        L = len(self.layers) - 1
        H = L - 1
        if mupc:
            d_in = F(self.layers[0].s)
            N = F(max(l.n for l in self.layers[:L - 1])) if H > 0 else F(self.layers[L - 1].n)
            for l in range(1, L + 1):
                if l == 1:
                    a = F(d_in ** F(-0.5))
                elif l == L:
                    a = F(1) / N
                else:
                    a = F((N * F(L)) ** F(-0.5))
                self.layers[l - 1].a = F(a)
        if residual:
            for l in range(2, H + 1):
                self.layers[l - 1].residual = True

    # ---------------------------------------------------------------- layer primitives
    def _zin(self, L):
        # SimplePCLayer feeds f(z) into the GEMM (src/layers/SimplePCLayer.cpp:149-150).
        return act(L.act, L.z) if self.kind == "simple" else L.z

    def compute_mu(self, L):
        """DirectKPPCLayer.cpp:267-310, FullPCLayer.cpp:246-298, SimplePCLayer.cpp:132-183."""
        if L.n == 0:
            return
        if L.clamped and L.cache_valid:
            L.mu[...] = L.cmu
            L.preact[...] = L.cpre
            return
        if self.kind == "simple":
            L.zF = self._zin(L)
            L.mu[...] = L.zF @ L.W.T + L.b
            L.preact[...] = L.mu
        else:
            L.preact[...] = (L.a * (L.z @ L.W.T)).astype(F) + L.b
            L.mu[...] = act(L.act, L.preact)
            if L.residual:
                L.mu += L.z
        if L.clamped:
            L.cmu[...] = L.mu
            L.cpre[...] = L.preact
            L.cache_valid = True

    def calculate_state(self, i, need_energy):
        """DirectKPPCLayer.cpp:243-265, FullPCLayer.cpp:210-244, SimplePCLayer.cpp:81-130."""
        L = self.layers[i]
        energy = 0.0
        if i == 0:
            L.e[...] = 0
        else:
            mu = self.layers[i - 1].mu
            if L.cross_entropy:
                L.e[...], en = softmax_ce(L.z, mu)
                energy = en if need_energy else 0.0
            else:
                L.e[...] = L.z - mu
                if need_energy:
                    energy = float(F(0.5) * (L.e * L.e).sum(dtype=F))
        self.compute_mu(L)
        return energy

    def update_state(self, i):
        """DirectKPPCLayer.cpp:318-359, FullPCLayer.cpp:300-380, SimplePCLayer.cpp:185-257."""
        L = self.layers[i]
        if L.clamped:
            return
        if i + 1 < len(self.layers) and L.n > 0:
            above = self.layers[i + 1]
            if self.kind == "simple":
                fb = above.e @ L.W
                L.z += L.ir * (fb * dact(L.act, L.z) - L.e)
                return
            if self.kind == "full" and above.cross_entropy and not above.clamped:
                L.z -= L.ir * L.e
                return
            fe = above.e * dact(L.act, L.preact)
            fb = (L.a * (fe @ L.W)).astype(F) - L.e
            if L.momentum is not None:
                L.v[...] = L.momentum * L.v
                L.v += (F(1) - L.momentum) * fb
                L.z += L.ir * L.v
            else:
                L.z += L.ir * fb
            if L.residual:
                L.z += L.ir * above.e
        else:
            L.z -= L.ir * L.e

    def update_weights(self, i):
        """DirectKPPCLayer.cpp:361-501, FullPCLayer.cpp:382-512, SimplePCLayer.cpp:259-350."""
        L = self.layers[i]
        if i + 1 >= len(self.layers) or L.n == 0:
            return
        above = self.layers[i + 1]
        term_e = self.layers[-1].e if self.e_terminal is None else self.e_terminal
        B = F(self.global_B or self.B)
        if self.kind == "simple":
            g, zin, a = above.e, L.zF, F(1)
        else:
            g, zin, a = above.e * dact(L.act, L.preact), L.z, L.a
        # raw sums over the batch rows held here; a batch-sharded run sums them over the shards
        G, Gb = g.T @ zin, g.sum(axis=0, dtype=F)
        GP = None if self.kind == "simple" else L.z.T @ term_e
        if self.grad_sync is not None:
            G, Gb, GP = self.grad_sync("learn", i, [G, Gb, GP])
        if self.opt == "SGD":
            if L.lmbda > 0:
                L.W *= F(1) - L.lmbda
            L.W += F(a * L.lr / B) * G
            L.b += F(L.lr / B) * Gb
        else:
            L.t += 1
            gW = (F(-1) * a) * G
            gb = F(-1) * Gb
            adam_step(L.W, gW, L.mW, L.vW, L.t, L.lr,
                      wd=(L.lr * L.lmbda) if self.opt == "ADAMW" else None)
            adam_step(L.b, gb, L.mb, L.vb, L.t, L.lr)
        if self.kind == "simple":
            return
        flr = F(L.fl * a) if self.kind == "full" else L.fl
        if self.opt_psi == "SGD":
            if self.kind == "dkp" and self.psi_decay > 0:
                L.Psi *= F(1) - self.psi_decay
            L.Psi += F(flr / B) * GP
        else:
            L.tP += 1
            gP = F(-1) * GP
            wd = None
            if self.opt_psi == "ADAMW":
                dec = self.psi_decay if (self.kind == "dkp" and self.psi_decay >= 0) else L.lmbda
                wd = flr * dec
            adam_step(L.Psi, gP, L.mP, L.vP, L.tP, flr, wd=wd)

    def dfa(self, i):
        """DirectKPPCLayer.cpp:503-549, FullPCLayer.cpp:514-572."""
        L = self.layers[i]
        if i + 1 >= len(self.layers) or getattr(self.layers[i + 1], "Psi", None) is None:
            return
        above = self.layers[i + 1]
        term_e = self.layers[-1].e if self.e_terminal is None else self.e_terminal
        proj = (term_e @ above.Psi.T) * dact(L.act, L.preact)
        G = proj.T @ L.z
        if self.grad_sync is not None:
            G, = self.grad_sync("dfa", i, [G])
        if self.kind == "full" and L.lmbda > 0 and L.fl != 0:
            L.W *= F(1) - L.lmbda
        L.W += F(L.fl * L.a / F(self.global_B or self.B)) * G

    # ---------------------------------------------------------------- network phases
    def reset(self):
        for L in self.layers:
            L.z[...] = 0
            if self.kind == "full":  # FullPCLayer.cpp:664-671
                L.e[...] = 0
                if L.v is not None:
                    L.v[...] = 0

    def clamp(self, i, data):
        L = self.layers[i]
        L.z[...] = np.asarray(data, F).reshape(L.z.shape)
        L.clamped, L.cache_valid = True, False

    def project_forward(self):
        """DirectKPPCNetwork.cpp:349-371, SimplePCNetwork.cpp:162-177."""
        for i in range(len(self.layers) - 1):
            self.compute_mu(self.layers[i])
            if not self.layers[i + 1].clamped:
                self.layers[i + 1].z[...] = self.layers[i].mu

    def step(self):
        """Jacobi settling step, DirectKPPCNetwork.cpp:429-439."""
        for i in range(len(self.layers)):
            self.calculate_state(i, False)
        for i in range(len(self.layers)):
            self.update_state(i)

    def epc_step(self):
        """src/networks/FullPCNetwork.cpp:99-131."""
        Ls = self.layers
        self.compute_mu(Ls[0])
        for i in range(1, len(Ls) - 1):
            Ls[i].z[...] = Ls[i - 1].mu + Ls[i].e  # ReconstructBelief, FullPCLayer.cpp:574-582
            self.compute_mu(Ls[i])
        self.calculate_state(len(Ls) - 1, False)
        adj, scale = Ls[-1].e, F(-1)
        for i in range(len(Ls) - 2, 0, -1):
            L = Ls[i]
            fe = adj * dact(L.act, L.preact)
            L.adj[...] = (L.a * scale) * (fe @ L.W)
            if L.residual:
                L.adj += scale * adj
            if not L.clamped:  # UpdateErrorEPC, FullPCLayer.cpp:632-640
                L.e *= F(1) - L.ir
                L.e -= L.ir * L.adj
            adj, scale = L.adj, F(1)

    def learn(self):
        """Refresh preact/mu from the settled z, then update (DirectKPPCNetwork.cpp:481-495)."""
        n = len(self.layers)
        if self.kind != "simple":
            for i in range(n - 1):
                self.compute_mu(self.layers[i])
        for i in range(n - 1):
            self.update_weights(i)
        if self.center:
            for i in range(n - 1):
                center_rows(self.layers[i].W)

    def final_energy(self):
        return float(sum(F(self.calculate_state(i, True)) for i in range(len(self.layers))))

    # ---------------------------------------------------------------- entry points
    def train_step(self, x, y, T):
        """DirectKPPCNetwork.cpp:513-603 / FullPCNetwork.cpp:134-251 /
        SimplePCNetwork.cpp:85-104 (C++ TrainStep)."""
        self.reset()
        self.clamp(0, x)
        self.clamp(len(self.layers) - 1, y)
        n = len(self.layers)
        if self.kind == "simple":
            for _ in range(T):
                for i in range(n):
                    self.calculate_state(i, False)
                for i in range(n):
                    self.update_state(i)
            energy = self.final_energy()
            self.learn()
        elif self.kind == "dkp":
            self.project_forward()
            self.calculate_state(n - 1, False)
            for i in range(n - 1):
                self.dfa(i)
            for _ in range(T):
                self.step()
            self.learn()
            energy = self.final_energy()
        else:
            self.project_forward()
            self.calculate_state(n - 1, False)
            for _ in range(T):
                self.epc_step() if self.epc else self.step()
                if self.ipc:
                    self.learn()
                    for L in self.layers:
                        L.cache_valid = False
            for i in range(n - 1):  # FullPCNetwork.cpp:72-82
                self.compute_mu(self.layers[i])
            for i in range(n - 1):
                self.dfa(i)
            if not self.ipc:
                self.learn()
            energy = self.final_energy()
        self.layers[-1].clamped = False
        return energy

    def train_step_with_projection(self, x, y, T, compute_energy=True):
        """SimplePCNetwork.cpp:179-252 (CPU branch)."""
        n = len(self.layers)
        self.reset()
        self.clamp(0, x)
        self.clamp(n - 1, y)
        self.project_forward()
        for _ in range(T):
            for i in range(n):
                self.calculate_state(i, False)
            for i in range(n):
                self.update_state(i)
        self.learn()
        energy = sum(F(self.calculate_state(i, compute_energy)) for i in range(n))
        self.layers[-1].clamped = False
        return float(energy) if compute_energy else 0.0

    def train_step_python(self, x, y, T):
        """deepity/SimplePCN.py:269-293: the Python-level SimplePCN.train_step loop; returns
        the SUM of the per-step energies."""
        n = len(self.layers)
        self.reset()
        self.clamp(0, x)
        self.clamp(n - 1, y)
        total = F(0)
        for _ in range(T):
            total += F(sum(F(self.calculate_state(i, True)) for i in range(n)))
            for i in range(n):
                self.update_state(i)
        self.learn()
        self.layers[-1].clamped = False
        return float(total)

    def predict(self, x, T, with_projection=None):
        """DirectKPPCNetwork.cpp:605-668 (always projects); SimplePCNetwork.cpp:106-160
        (plain) and :254-312 (with projection)."""
        n = len(self.layers)
        if with_projection is None:
            with_projection = self.kind != "simple"
        self.reset()
        self.clamp(0, x)
        if with_projection:
            self.project_forward()
        for _ in range(T):
            if self.kind == "full" and self.epc:
                self.epc_step()
            else:
                self.step()
        if self.kind == "full" and self.layers[-1].cross_entropy:  # FullPCNetwork.cpp:285-291
            self.compute_mu(self.layers[-2])
            self.layers[-1].z[...] = self.layers[-2].mu
        return self.layers[-1].z.copy()

    def get(self, layer, name):
        L = self.layers[layer]
        return np.asarray(getattr(L, {"weight.m": "mW", "weight.v": "vW", "bias.m": "mb",
                                      "bias.v": "vb", "psi.m": "mP", "psi.v": "vP"}.get(name, name)))

    def set(self, layer, name, value):
        a = getattr(self.layers[layer], name)
        a[...] = np.asarray(value, F).reshape(a.shape)

"""CPU restatement (numpy) of the reference's convolutional predictive-coding path.

Test infrastructure only: nothing under deepity_b200/ imports this module.  It follows
src/layers/SimpleConvPCLayer.cpp and src/networks/SimpleConvPCNetwork.cpp (CPU branch) phase by
phase, with the convolution written as the reference writes it: im2col columns
(include/deepity/utils/Im2Col.h:78-152) times W[outC, inC*kH*kW], feedback as W^T times the
gated error followed by col2im (Im2Col.h:182-259).  Pinned by tests/test_conv_oracle_pin.py
against outputs of the compiled reference (tests/golden/conv_*.npz).
"""
from __future__ import annotations

import numpy as np

from .pc_oracle import F, act, adam_step, center_rows, dact


def conv_out_dim(n, k, s, p):
    """include/deepity/utils/Im2Col.h:47-50."""
    return (n + 2 * p - k) // s + 1


def im2col(x, kH, kW, sH, sW, pH, pW):
    """x [B,C,H,W] -> cols [B, C*kH*kW, oH*oW]; row index (c*kH+ky)*kW+kx."""
    B, C, H, W = x.shape
    oH, oW = conv_out_dim(H, kH, sH, pH), conv_out_dim(W, kW, sW, pW)
    xp = np.zeros((B, C, H + 2 * pH, W + 2 * pW), F)
    xp[:, :, pH:pH + H, pW:pW + W] = x
    cols = np.empty((B, C, kH, kW, oH, oW), F)
    for ky in range(kH):
        for kx in range(kW):
            cols[:, :, ky, kx] = xp[:, :, ky:ky + sH * oH:sH, kx:kx + sW * oW:sW]
    return cols.reshape(B, C * kH * kW, oH * oW)


def col2im(cols, C, H, W, kH, kW, sH, sW, pH, pW):
    """Adjoint of im2col: accumulates cols [B, C*kH*kW, oH*oW] into [B,C,H,W]."""
    B = cols.shape[0]
    oH, oW = conv_out_dim(H, kH, sH, pH), conv_out_dim(W, kW, sW, pW)
    c6 = cols.reshape(B, C, kH, kW, oH, oW)
    xp = np.zeros((B, C, H + 2 * pH, W + 2 * pW), F)
    for ky in range(kH):
        for kx in range(kW):
            xp[:, :, ky:ky + sH * oH:sH, kx:kx + sW * oW:sW] += c6[:, :, ky, kx]
    return xp[:, :, pH:pH + H, pW:pW + W].copy()


class ConvLayer:
    def __init__(self, B, d, lr, ir, lmbda):
        self.B = B
        self.C, self.O, self.H, self.W_ = d["inC"], d["outC"], d["H"], d["W"]
        self.kH, self.kW, self.sH, self.sW = d["kH"], d["kW"], d["sH"], d["sW"]
        self.pH, self.pW = d["pH"], d["pW"]
        self.act = d["act"]
        self.lr, self.ir, self.lmbda = F(lr), F(ir), F(lmbda)
        self.z = np.zeros((B, self.C, self.H, self.W_), F)
        self.e = np.zeros_like(self.z)
        self.clamped = self.cache_valid = False
        if self.O > 0:
            self.oH = conv_out_dim(self.H, self.kH, self.sH, self.pH)
            self.oW = conv_out_dim(self.W_, self.kW, self.sW, self.pW)
            rows = self.C * self.kH * self.kW
            self.W = np.zeros((self.O, rows), F)
            self.b = np.zeros(self.O, F)
            # `mu` is one buffer that holds the prediction after ComputeMuOnly and the
            # activation derivative after UpdateState (SimpleConvPCLayer.cpp:312-316,339).
            self.mu = np.zeros((B, self.O, self.oH * self.oW), F)
            self.preact = np.zeros_like(self.mu)
            self.mW, self.vW = np.zeros_like(self.W), np.zeros_like(self.W)
            self.mb, self.vb = np.zeros_like(self.b), np.zeros_like(self.b)
            self.t = 0

    def cols(self):
        return im2col(self.z, self.kH, self.kW, self.sH, self.sW, self.pH, self.pW)


class ConvOracle:
    """SimpleConvPCNetwork on the CPU.  ``layers`` as for oracle.ref.RefConvNet."""

    def __init__(self, layers, batch, lr, ir, lmbda, optimizer="SGD", center_weights=False):
        self.B = batch
        self.layers = [ConvLayer(batch, d, lr, ir, lmbda) for d in layers]
        self.opt, self.center = optimizer, center_weights

    # ----------------------------------------------------------------- layer phases
    def compute_mu(self, L):
        """SimpleConvPCLayer::ComputeMuOnly, SimpleConvPCLayer.cpp:214-300."""
        if L.O == 0:
            return
        if L.clamped and L.cache_valid:
            L.mu[...] = L.cmu
            L.preact[...] = L.cpre
            return
        pre = np.einsum("ok,bkn->bon", L.W, L.cols(), dtype=F, optimize=True).astype(F)
        pre += L.b[None, :, None]
        L.preact[...] = pre
        L.mu[...] = act(L.act, pre)
        if L.clamped:
            L.cmu, L.cpre = L.mu.copy(), L.preact.copy()
            L.cache_valid = True

    def calculate_state(self, i, need_energy):
        """SimpleConvPCLayer::CalculateState, SimpleConvPCLayer.cpp:188-212."""
        L = self.layers[i]
        energy = F(0)
        if i == 0:
            L.e[...] = 0
        else:
            L.e[...] = L.z - self.layers[i - 1].mu.reshape(L.z.shape)
            if need_energy:
                energy = F(0.5) * F((L.e * L.e).sum(dtype=F))
        self.compute_mu(L)
        return energy

    def update_state(self, i):
        """SimpleConvPCLayer::UpdateState, SimpleConvPCLayer.cpp:302-400."""
        L = self.layers[i]
        if L.O > 0:
            L.mu[...] = dact(L.act, L.preact)
        if L.clamped:
            return
        dz = np.zeros_like(L.z)
        if i + 1 < len(self.layers) and L.O > 0:
            g = self.layers[i + 1].e.reshape(L.mu.shape) * L.mu
            back = np.einsum("ok,bon->bkn", L.W, g, dtype=F, optimize=True).astype(F)
            dz = col2im(back, L.C, L.H, L.W_, L.kH, L.kW, L.sH, L.sW, L.pH, L.pW)
        dz -= L.e
        L.z += L.ir * dz

    def update_weights(self, i):
        """SimpleConvPCLayer::UpdateWeights, SimpleConvPCLayer.cpp:402-560."""
        L = self.layers[i]
        if i + 1 >= len(self.layers) or L.O == 0:
            return
        g = self.layers[i + 1].e.reshape(L.mu.shape) * L.mu
        G = np.einsum("bon,bkn->ok", g, L.cols(), dtype=F, optimize=True).astype(F)
        Gb = g.sum(axis=(0, 2), dtype=F)
        B = F(self.B)
        if self.opt == "SGD":
            if L.lmbda > 0:
                L.W *= F(1) - L.lmbda
            L.W += F(L.lr / B) * G
            L.b += F(L.lr / B) * Gb
        else:
            L.t += 1
            gs = F(-1) / B
            adam_step(L.W, gs * G, L.mW, L.vW, L.t, L.lr,
                      wd=(L.lr * L.lmbda) if self.opt == "ADAMW" else None)
            adam_step(L.b, gs * Gb, L.mb, L.vb, L.t, L.lr)

    # ----------------------------------------------------------------- network
    def reset(self):
        for L in self.layers:
            L.z[...] = 0

    def clamp(self, i, data):
        L = self.layers[i]
        L.z[...] = np.asarray(data, F).reshape(L.z.shape)
        L.clamped, L.cache_valid = True, False

    def project_forward(self):
        """SimpleConvPCNetwork::ProjectForward."""
        for i in range(len(self.layers) - 1):
            self.compute_mu(self.layers[i])
            if not self.layers[i + 1].clamped:
                self.layers[i + 1].z[...] = self.layers[i].mu.reshape(self.layers[i + 1].z.shape)

    def settle(self, T):
        n = len(self.layers)
        for _ in range(T):
            for i in range(n):
                self.calculate_state(i, False)
            for i in range(n):
                self.update_state(i)

    def learn(self):
        for i in range(len(self.layers) - 1):
            self.update_weights(i)
        if self.center:
            for L in self.layers[:-1]:
                center_rows(L.W)

    def train_step(self, x, y, T, with_projection=False):
        """SimpleConvPCNetwork::TrainStep / TrainStepWithProjection (CPU branch)."""
        n = len(self.layers)
        self.reset()
        self.clamp(0, x)
        self.clamp(n - 1, y)
        if with_projection:
            self.project_forward()
        self.settle(T)
        self.learn()
        energy = float(sum(F(self.calculate_state(i, True)) for i in range(n)))
        self.layers[-1].clamped = False
        return energy

    def predict(self, x, T, with_projection=False):
        self.reset()
        self.clamp(0, x)
        if with_projection:
            self.project_forward()
        self.settle(T)
        return self.layers[-1].z.reshape(self.B, -1).copy()

    def get(self, layer, name):
        return np.asarray(getattr(self.layers[layer], name))

    def set(self, layer, name, value):
        a = getattr(self.layers[layer], name)
        a[...] = np.asarray(value, F).reshape(a.shape)

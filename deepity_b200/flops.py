"""Algorithmic FLOP count of one train step (GEMM terms only).

The same formula as ``dpcn_train_step_flops`` of the C ABI, for networks that exist only as
a list of widths (a layer-sharded network counts the whole stack, not one rank's block).
"""
from __future__ import annotations

from typing import Sequence


def algorithmic_flops(kind: str, sizes: Sequence[int], batch: int, steps: int) -> float:
    """GEMM FLOPs one train step needs under the reference's CPU semantics (2*M*N*K each).

    Per weight layer: T+3 (DirectKP), T+4 (Full) or T+1 (Simple) forward products, T feedback
    products and the weight-shaped products (learn, plus the direct-feedback update when the
    layer above owns feedback weights), plus the skinny Psi / projection products.  The
    clamped input layer evaluates its prediction once and is never updated."""
    n, B, T = len(sizes), float(batch), steps
    total = 0.0
    for i in range(n - 1):
        s, nx, ts = sizes[i], sizes[i + 1], sizes[-1]
        g = 2.0 * B * s * nx
        if kind == "simple":
            fwd, fb, wg = T + 1, T, 1
        else:
            fwd, fb, wg = (T + 3 if kind == "dkp" else T + 4), T, (2 if i + 2 < n else 1)
            total += 2.0 * B * s * ts + (2.0 * B * nx * ts if i + 2 < n else 0.0)
        if i == 0:
            fwd, fb = 1, 0
        total += g * (fwd + fb + wg)
    return total

"""Generate the golden fixtures under tests/golden/ from the compiled reference.

    python tests/golden/make_golden.py

Needs oracle/_ref/libdeepity_ref.so (python oracle/build_ref.py, which needs the reference
checkout).  Each fixture stores the case description (from which tests/common.make_case
regenerates the seeded inputs bit-for-bit), the energy of every train step, the prediction
after training, and the tensors of the network after the last step — in full for small
networks, as per-tensor float64 sums / sums of squares for the two benchmark-shaped ones.
The reference has no golden vectors of its own for a whole train step, so these are its own
outputs on this machine's OpenBLAS.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from common import make_case, state_names  # noqa: E402
from oracle.ref import RefNet  # noqa: E402

CASES = {
    "dkp_tanh_small": dict(kind="dkp", sizes=[16, 32, 32, 32, 10], batch=8, T=2, steps=3,
                           hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "dkp_relu_center_decay": dict(kind="dkp", sizes=[50, 24, 24, 10], batch=12, T=3, steps=3,
                                  hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="relu"),
                                  options=dict(center_weights=1, psi_decay=0.01)),
    "dkp_adamw_psi_adam": dict(kind="dkp", sizes=[20, 48, 48, 10], batch=16, T=2, steps=3,
                               hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.01, act="gelu"),
                               options=dict(optimizer="ADAMW", psi_optimizer="ADAM")),
    "dkp_c2_shape": dict(kind="dkp", sizes=[784] + [256] * 8 + [10], batch=256, T=2, steps=2,
                         x_dist="uniform", stats_only=True,
                         hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh")),
    "simple_sigmoid_small": dict(kind="simple", sizes=[40, 24, 24, 10], batch=8, T=6, steps=3,
                                 x_dist="uniform", mode="python",
                                 hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="sigmoid")),
    "simple_c1_shape": dict(kind="simple", sizes=[784, 128, 128, 10], batch=64, T=20, steps=2,
                            x_dist="uniform", mode="python", stats_only=True,
                            hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="sigmoid")),
    "simple_projection_adam": dict(kind="simple", sizes=[30, 40, 10], batch=16, T=5, steps=3,
                                   mode="projection",
                                   hyper=dict(lr=1e-3, ir=0.1, lmbda=0.0, act="tanh"),
                                   options=dict(optimizer="ADAM")),
    "full_gelu_ce_adam": dict(kind="full", sizes=[30, 40, 40, 40, 10], batch=16, T=4, steps=3,
                              hyper=dict(lr=1e-3, ir=0.1, fl=1e-4, lmbda=0.0, act="gelu"),
                              options=dict(cross_entropy=1, optimizer="ADAM",
                                           psi_optimizer="ADAM")),
    "full_mupc_residual_momentum": dict(kind="full", sizes=[30, 40, 40, 40, 10], batch=16, T=4,
                                        steps=3,
                                        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01,
                                                   act="tanh"),
                                        options=dict(mupc=1, residual=1, momentum=0.9)),
    "full_ipc": dict(kind="full", sizes=[30, 40, 40, 10], batch=16, T=3, steps=2,
                     hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh"),
                     options=dict(ipc=1)),
    # a shape the tensor-core kernels take (square layers of width 512, batch 1024: CTA-pair
    # tiles, the persistent forward sweep), so that path meets reference output directly
    "dkp_tensor_run_shape": dict(kind="dkp", sizes=[512] + [512] * 12 + [10], batch=1024, T=2,
                                 steps=2, stats_only=True,
                                 hyper=dict(lr=1e-2, ir=0.1, fl=1e-2, lmbda=0.0, act="tanh")),
}


def run_reference(case):
    kind, sizes, B, T = case["kind"], case["sizes"], case["batch"], case["T"]
    params, x, y = make_case(kind, sizes, B, seed=case.get("seed", 0),
                             x_dist=case.get("x_dist", "normal"))
    opts = {}
    for k, v in case.get("options", {}).items():
        if k == "psi_decay":
            opts[k] = (1, v)
        elif k == "momentum":
            opts[k] = (1, v)
        else:
            opts[k] = v
    hyper = dict(case["hyper"])
    if kind == "simple":
        hyper["fl"] = 0.0
    net = RefNet(kind, sizes, B, options=opts, **hyper)
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set(l, name, v)
    energies = []
    for _ in range(case["steps"]):
        mode = case.get("mode", "train_step")
        if mode == "python":  # deepity/SimplePCN.py:269-293
            net.phase("reset")
            net.phase("clamp_x", x)
            net.phase("clamp_y", y)
            e = 0.0
            for _t in range(T):
                e += net.phase("calculate_state_energy")
                net.phase("update_state")
            net.phase("update_weights")
            net.phase("unclamp_y")
        elif mode == "projection":
            e = net.train_step_with_projection(x, y, T)
        else:
            e = net.train_step(x, y, T)
        energies.append(e)
    out = {"energies": np.asarray(energies, dtype=np.float64)}
    for l in range(net.num_layers):
        for name in state_names(kind):
            a = net.get(l, name)
            if a.size == 0:
                continue
            if case.get("stats_only"):
                a64 = a.astype(np.float64)
                out[f"stat.{l}.{name}"] = np.asarray([a64.sum(), (a64 * a64).sum()])
            else:
                out[f"t.{l}.{name}"] = a
    out["predict"] = net.predict(x, T, with_projection=(kind != "simple" or
                                                        case.get("mode") == "projection"))
    return out


def main():
    only = set(sys.argv[1:])  # optional: names of the fixtures to (re)generate
    for name, case in CASES.items():
        if only and name not in only:
            continue
        out = run_reference(case)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "energies", out["energies"])
    with open(os.path.join(HERE, "cases.json"), "w") as f:
        json.dump(CASES, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()

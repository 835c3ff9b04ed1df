"""Shared helpers of the parity tests: seeded cases, oracle construction, comparison."""
from __future__ import annotations

import numpy as np

from oracle.pc_oracle import PCOracle

KINDS = {"simple": 0, "dkp": 1, "full": 2}

# Parity bound for the fp32 path against the CPU oracle: per tensor,
# max|a-b| <= TOL * max(1, max|ref|).  Adam-type updates divide by sqrt(v)+eps with v ~ g^2,
# which turns rounding-level gradient differences into differences of up to one step
# (lr) per element; those cases use the looser ADAM_TOL (the compiled reference and its numpy
# restatement differ by 7e-5 on them already).
TOL = 1e-4
ADAM_TOL = 5e-4
# The single-pass TF32 mode is judged at the reference's own CPU-vs-GPU bound
# (tests/tDirectKPBatchedGPUVerify.cpp:47-58 in the reference).
TF32_TOL = 1e-2


def make_case(kind, sizes, batch, seed=0, x_dist="normal", bias_scale=0.1):
    """Seeded weights and one batch for a network of the given widths."""
    rng = np.random.default_rng(seed)
    ts = sizes[-1]
    params = []
    for l in range(len(sizes) - 1):
        s, n = sizes[l], sizes[l + 1]
        p = {"W": rng.normal(0, np.sqrt(2 / (s + n)), (n, s)).astype(np.float32),
             "b": rng.normal(0, bias_scale, n).astype(np.float32)}
        if kind != "simple":
            p["Psi"] = rng.normal(0, np.sqrt(2 / (s + ts)), (s, ts)).astype(np.float32)
        params.append(p)
    if x_dist == "uniform":
        x = rng.random((batch, sizes[0]), dtype=np.float32)
    else:
        x = rng.normal(size=(batch, sizes[0])).astype(np.float32)
    y = np.eye(ts, dtype=np.float32)[rng.integers(0, ts, batch)]
    return params, x, y


def load_params(net, params):
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set(l, name, v)


def make_oracle(kind, sizes, batch, params, **kw):
    orc = PCOracle(kind, sizes, batch, **kw)
    load_params(orc, params)
    return orc


def rel_err(ref, got):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    got = np.asarray(got, dtype=np.float64).ravel()
    assert ref.shape == got.shape, (ref.shape, got.shape)
    if ref.size == 0:
        return 0.0
    return float(np.abs(ref - got).max() / max(1.0, np.abs(ref).max()))


def rel_err_of_update(ref, got, init):
    """Error of the UPDATE (after - initial) relative to the largest update element.  Weights
    are of order 0.1 and their per-step updates of order lr, so a bound relative to
    max(1, |W|) alone would also pass when the update is missing altogether."""
    init = np.asarray(init, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    d_ref = ref - init
    d_got = np.asarray(got, dtype=np.float64).ravel() - init
    if d_ref.size == 0:
        return 0.0
    # both sides store the parameter in fp32: a few ulps of the parameter itself are not an
    # error of the update
    slack = 4 * np.finfo(np.float32).eps * np.abs(ref).max()
    err = max(0.0, float(np.abs(d_ref - d_got).max()) - slack)
    scale = np.abs(d_ref).max()
    return err if scale == 0.0 else err / scale


# Bounds on the error of the parameter UPDATES (see rel_err_of_update), SGD cases only: an
# Adam-type step m/(sqrt(v)+eps) can flip by a whole step on a near-zero gradient element.
DELTA_TOL = 2e-3        # fp32 mode (CUDA cores, 3xTF32, 3xBF16)
DELTA_TOL_MIXED = 3e-2  # gradient products in one TF32 pass
DELTA_TOL_TF32 = 1e-1   # everything in one TF32 pass


def initial_parameters(case):
    """The seeded W, b, Psi a case starts from, keyed like the outputs ("t.<layer>.<name>")."""
    params, _, _ = make_case(case["kind"], case["sizes"], case["batch"], seed=case.get("seed", 0),
                             x_dist=case.get("x_dist", "normal"))
    return {f"t.{l}.{name}": np.asarray(v, dtype=np.float32).ravel()
            for l, p in enumerate(params) for name, v in p.items()}


def state_names(kind):
    return ["z", "e", "W", "b"] + ([] if kind == "simple" else ["Psi"])


# ------------------------------------------------------------------------------------------
# Running one golden-style case on the numpy oracle or on the GPU library.
# ------------------------------------------------------------------------------------------
def _oracle_kwargs(case):
    kw = dict(case["hyper"])
    for k, v in case.get("options", {}).items():
        kw[k] = bool(v) if k in ("center_weights", "cross_entropy", "mupc", "residual", "ipc", "epc") else v
    return kw


def run_oracle(case):
    kind, sizes, B, T = case["kind"], case["sizes"], case["batch"], case["T"]
    params, x, y = make_case(kind, sizes, B, seed=case.get("seed", 0),
                             x_dist=case.get("x_dist", "normal"))
    orc = make_oracle(kind, sizes, B, params, **_oracle_kwargs(case))
    mode = case.get("mode", "train_step")
    energies = []
    for _ in range(case["steps"]):
        if mode == "python":
            energies.append(orc.train_step_python(x, y, T))
        elif mode == "projection":
            energies.append(orc.train_step_with_projection(x, y, T))
        else:
            energies.append(orc.train_step(x, y, T))
    out = {"energies": np.asarray(energies, dtype=np.float64)}
    for l in range(len(orc.layers)):
        for name in state_names(kind):
            if name in ("W", "b", "Psi") and orc.layers[l].n == 0:
                continue
            out[f"t.{l}.{name}"] = np.array(orc.get(l, name), dtype=np.float32).ravel()
    out["predict"] = orc.predict(x, T, with_projection=(kind != "simple" or mode == "projection"))
    return out


def build_gpu_net(case, precision="fp32", use_graph=True, device="cuda"):
    """A deepity_b200 network for a golden-style case, with the case's seeded parameters."""
    import deepity_b200 as dp
    from deepity_b200.layer import Activation

    kind, sizes, B = case["kind"], case["sizes"], case["batch"]
    hy, opts = case["hyper"], case.get("options", {})
    acts = {"tanh": dp.TanH, "relu": dp.ReLU, "gelu": dp.GeLU, "sigmoid": dp.Sigmoid,
            "esigmoid": dp.ESigmoid, "hard_tanh": dp.HardTanH}
    arch = []
    for l in range(len(sizes) - 1):
        arch.append(dp.Linear(sizes[l], sizes[l + 1]))
        if hy["act"] != "linear":
            arch.append(acts[hy["act"]]())
    cls = {"simple": dp.SimplePCN, "dkp": dp.DKPPCN, "full": dp.FullPCN}[kind]
    net = cls(*arch, batch_size=B, device=device)
    kw = dict(learning_rate=hy["lr"], inference_rate=hy["ir"], lmbda=hy["lmbda"],
              optimizer=opts.get("optimizer", "SGD"), seed=1,
              center_weights=bool(opts.get("center_weights", 0)), precision=precision)
    if kind != "simple":
        kw.update(feedback_rate=hy["fl"], psi_optimizer=opts.get("psi_optimizer", "SGD"))
    if kind == "dkp":
        kw.update(psi_decay=opts.get("psi_decay"))
    if kind == "full":
        kw.update(use_mu_pc_scaling=bool(opts.get("mupc", 0)),
                  use_residual_connections=bool(opts.get("residual", 0)),
                  use_ipc=bool(opts.get("ipc", 0)), use_epc=bool(opts.get("epc", 0)), use_momentum="momentum" in opts,
                  momentum_beta=opts.get("momentum", 0.9),
                  use_cross_entropy=bool(opts.get("cross_entropy", 0)))
    if kind == "simple":
        kw.update(use_cross_entropy=bool(opts.get("cross_entropy", 0)))
    net.configure(**kw)
    net.set_use_graph(use_graph)
    params, x, y = make_case(kind, sizes, B, seed=case.get("seed", 0),
                             x_dist=case.get("x_dist", "normal"))
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set_tensor(l, name, v)
    return net, x, y


def run_gpu(case, precision="fp32", use_graph=True, staged_gradients=False):
    kind, T = case["kind"], case["T"]
    net, x, y = build_gpu_net(case, precision, use_graph)
    if staged_gradients:
        # the batch-sharded update path with a single shard: stage, "all-reduce", apply
        net.set_gradient_sync(lambda t: None, case["batch"])
    mode = case.get("mode", "train_step")
    energies = []
    for _ in range(case["steps"]):
        if kind == "simple" and mode == "python":
            energies.append(net.train_step(x, y, T))
        elif kind == "simple" and mode == "projection":
            energies.append(net.train_step_with_projection(x, y, T))
        elif kind == "simple":
            energies.append(net.train_step_native(x, y, T))
        else:
            energies.append(net.train_step(x, y, T))
    out = {"energies": np.asarray(energies, dtype=np.float64)}
    n_layers = len(case["sizes"])
    for l in range(n_layers):
        for name in state_names(kind):
            if name in ("W", "b", "Psi") and l == n_layers - 1:
                continue
            out[f"t.{l}.{name}"] = net.get_tensor(l, name)
    out["predict"] = net.predict(x, T, with_projection=(kind != "simple" or mode == "projection"))
    return out


def compare_outputs(ref, got, tol, what="", energy_tol=None, init=None, delta_tol=None):
    """ref may hold full tensors (t.*) or statistics (stat.*).  energy_tol: a separate bound
    for the energies where the reference's own fp32 accumulation is the limit.  init (from
    initial_parameters) with delta_tol: the parameter updates themselves are compared too."""
    worst = 0.0
    bad = []
    if init is not None:
        worst_delta = 0.0
        for k, w0 in init.items():
            if k in ref and k in got:
                err = rel_err_of_update(ref[k], got[k], w0)
                worst_delta = max(worst_delta, err)
                if not err <= delta_tol:
                    bad.append((k + " (update)", err))
        print(f"{what}: worst relative error of a parameter update {worst_delta:.2e}")
    for k, r in ref.items():
        if k == "energies":
            err = float(np.max(np.abs(r - got[k]) / np.maximum(1.0, np.abs(r))))
        elif k.startswith("stat."):
            g = np.asarray(got["t." + k[5:]], dtype=np.float64)
            gs = np.asarray([g.sum(), (g * g).sum()])
            # sums over n elements: compare relative to the L1 / L2 scale of the tensor
            scale = np.asarray([max(1.0, np.sqrt(r[1] * g.size)), max(1.0, r[1])])
            err = float(np.max(np.abs(r - gs) / scale))
        else:
            err = rel_err(r, got[k])
        worst = max(worst, err)
        if not err <= (energy_tol if (k == "energies" and energy_tol) else tol):
            bad.append((k, err))
    assert not bad, f"{what}: beyond tolerance {tol}: {bad[:8]}"
    return worst

"""Helpers shared by the convolutional tests: case descriptions, seeded inputs, and one
runner per implementation (numpy oracle, compiled reference, GPU library)."""
import numpy as np


def spec(inC, outC, H, W, kH=1, kW=1, sH=1, sW=1, pH=0, pW=0, act="linear"):
    return dict(inC=inC, outC=outC, H=H, W=W, kH=kH, kW=kW, sH=sH, sW=sW, pH=pH, pW=pW, act=act)


def chain(input_shape, convs, act):
    """convs: list of (outC, kH, kW, sH, sW, pH, pW); returns the layer specs including the
    terminal layer (outC = 0)."""
    c, h, w = input_shape
    layers = []
    for i, (o, kh, kw, sh, sw, ph, pw) in enumerate(convs):
        a = act if i + 1 < len(convs) else "linear"
        layers.append(spec(c, o, h, w, kh, kw, sh, sw, ph, pw, a))
        c, h, w = o, (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    layers.append(spec(c, 0, h, w))
    return layers


def make_conv_case(case):
    """Seeded W, b per weight layer and one batch (x ~ N(0,1) NCHW, y one-hot when the terminal
    layer is 1x1, else N(0,1))."""
    layers, B = case["layers"], case["batch"]
    rng = np.random.default_rng(case.get("seed", 0))
    params = []
    for d in layers[:-1]:
        rows = d["inC"] * d["kH"] * d["kW"]
        params.append({"W": rng.normal(0, np.sqrt(2.0 / rows), (d["outC"], rows)).astype(np.float32),
                       "b": rng.normal(0, 0.1, d["outC"]).astype(np.float32)})
    first, last = layers[0], layers[-1]
    x = rng.normal(size=(B, first["inC"], first["H"], first["W"])).astype(np.float32)
    if last["H"] == 1 and last["W"] == 1:
        y = np.eye(last["inC"], dtype=np.float32)[rng.integers(0, last["inC"], B)]
    else:
        y = rng.normal(size=(B, last["inC"] * last["H"] * last["W"])).astype(np.float32)
    return params, x, y


def _collect(net, case, energies, predict, stats=False):
    out = {"energies": np.asarray(energies, dtype=np.float64), "predict": np.asarray(predict).ravel()}
    for l, d in enumerate(case["layers"]):
        for name in ("z", "e") + (("W", "b") if d["outC"] > 0 else ()):
            a = np.array(net(l, name), dtype=np.float32).ravel()
            if stats:
                a64 = a.astype(np.float64)
                out[f"stat.{l}.{name}"] = np.asarray([a64.sum(), (a64 * a64).sum()])
            else:
                out[f"t.{l}.{name}"] = a
    return out


def _drive(net, case):
    params, x, y = make_conv_case(case)
    for l, p in enumerate(params):
        for name, v in p.items():
            net.set(l, name, v)
    proj = bool(case.get("projection", 0))
    energies = [net.train_step(x, y, case["T"], proj) for _ in range(case["steps"])]
    return energies, net.predict(x, case["T"], proj)


def run_conv_oracle(case):
    from oracle.conv_oracle import ConvOracle
    hy = case["hyper"]
    net = ConvOracle(case["layers"], case["batch"], hy["lr"], hy["ir"], hy["lmbda"],
                     case.get("optimizer", "SGD"), bool(case.get("center_weights", 0)))
    energies, pred = _drive(net, case)
    return _collect(net.get, case, energies, pred)


def run_conv_reference(case, device="cpu"):
    """device="gpu": the reference's own device path on whatever backend plugin its loader finds."""
    from oracle.ref import RefConvNet
    hy = case["hyper"]
    net = RefConvNet(case["layers"], case["batch"], hy["lr"], hy["ir"], hy["lmbda"],
                     case.get("optimizer", "SGD"), bool(case.get("center_weights", 0)),
                     device=device)
    energies, pred = _drive(net, case)
    # only the fixtures are reduced to statistics; the implementations under test return tensors
    return _collect(net.get, case, energies, pred, stats=bool(case.get("stats_only")))


def build_conv_gpu_net(case, use_graph=True):
    import deepity_b200 as dp
    acts = {"tanh": dp.TanH, "relu": dp.ReLU, "gelu": dp.GeLU, "sigmoid": dp.Sigmoid}
    layers = case["layers"]
    arch = []
    for d in layers:
        arch.append(dp.Convolution(d["outC"], d["kH"], d["kW"], d["sH"], d["sW"], d["pH"], d["pW"]))
        if d["act"] != "linear":
            arch.append(acts[d["act"]]())
    first = layers[0]
    net = dp.SimpleConvolutionalPCN(*arch, input_shape=(first["inC"], first["H"], first["W"]),
                                    batch_size=case["batch"])
    hy = case["hyper"]
    net.configure(learning_rate=hy["lr"], inference_rate=hy["ir"], lmbda=hy["lmbda"],
                  optimizer=case.get("optimizer", "SGD"),
                  center_weights=bool(case.get("center_weights", 0)), seed=1)
    net.set_use_graph(use_graph)
    return net


def run_conv_gpu(case, use_graph=True):
    net = build_conv_gpu_net(case, use_graph)

    class _Adapter:
        def set(self, l, name, v):
            net.set_tensor(l, name, v)

        def train_step(self, x, y, T, proj):
            return net.train_step_with_projection(x, y, T) if proj else net.train_step(x, y, T)

        def predict(self, x, T, proj):
            return net.predict_with_projection(x, T) if proj else net.predict(x, T)
    energies, pred = _drive(_Adapter(), case)
    return _collect(net.get_tensor, case, energies, pred)


CONV_CASES = {
    "conv_relu_small": dict(layers=chain((3, 8, 8), [(8, 3, 3, 2, 2, 1, 1), (16, 3, 3, 2, 2, 1, 1),
                                                     (10, 2, 2, 1, 1, 0, 0)], "relu"),
                            batch=4, T=3, steps=3, hyper=dict(lr=0.01, ir=0.1, lmbda=0.0)),
    "conv_adamw_center_projection": dict(
        layers=chain((3, 8, 8), [(8, 3, 3, 2, 2, 1, 1), (16, 3, 3, 2, 2, 1, 1),
                                 (10, 2, 2, 1, 1, 0, 0)], "tanh"),
        batch=4, T=3, steps=3, projection=1, optimizer="ADAMW", center_weights=1,
        hyper=dict(lr=1e-3, ir=0.1, lmbda=0.01)),
    # the shape of the reference's own sanity test (tests/tSimpleConvPCNetworkTrainStepSanity.cpp)
    "conv_tanh_sanity_shape": dict(layers=chain((1, 4, 4), [(2, 3, 3, 1, 1, 0, 0)], "tanh")[:1]
                                   + [spec(2, 0, 2, 2)],
                                   batch=1, T=5, steps=4, hyper=dict(lr=1e-3, ir=0.1, lmbda=0.0)),
    "conv_zero_steps": dict(layers=chain((3, 8, 8), [(8, 3, 3, 2, 2, 1, 1), (10, 4, 4, 1, 1, 0, 0)],
                                         "relu"),
                            batch=4, T=0, steps=3, hyper=dict(lr=0.01, ir=0.1, lmbda=0.01)),
    "conv_ragged_geometry": dict(layers=chain((2, 7, 9), [(5, 3, 2, 2, 1, 1, 0), (3, 2, 3, 1, 2, 0, 1),
                                                          (4, 3, 3, 1, 1, 0, 0)], "sigmoid"),
                                 batch=3, T=4, steps=3, optimizer="ADAM",
                                 hyper=dict(lr=1e-3, ir=0.1, lmbda=0.0)),
    # the benchmark shape: 32x32x3 -> 32 -> 64 -> 128 channels (3x3, stride 2, pad 1), 2048 -> 10
    "conv_c5_shape": dict(layers=chain((3, 32, 32), [(32, 3, 3, 2, 2, 1, 1), (64, 3, 3, 2, 2, 1, 1),
                                                     (128, 3, 3, 2, 2, 1, 1), (10, 4, 4, 1, 1, 0, 0)],
                                       "relu"),
                          # The reference adds the ~1.5 M squared errors of this shape in fp32, one
                          # after the other per thread: its energy is 8e-5 below the exactly
                          # summed value of its own error tensors, so energies get 5e-4 here.
                          batch=128, T=10, steps=2, stats_only=True, energy_tol=5e-4,
                          hyper=dict(lr=1e-3, ir=0.1, lmbda=0.0)),
}

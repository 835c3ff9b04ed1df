"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Every case runs K train steps on identical seeded inputs and explicitly set W/b/Psi and
compares the energy of every step, every layer's z and e after the last step, the updated
W, b and Psi, and a prediction — against the golden fixtures (outputs of the reference's own
CPU code) and against the numpy oracle run live.  Bound: common.TOL (1e-4 relative per
tensor) for the fp32 path, common.ADAM_TOL where an Adam-type optimizer is on.
"""
import json
import os

import numpy as np
import pytest

from common import (ADAM_TOL, DELTA_TOL, DELTA_TOL_MIXED, DELTA_TOL_TF32, TF32_TOL, TOL,
                    compare_outputs, initial_parameters, run_gpu, run_oracle)

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = json.load(open(os.path.join(GOLDEN, "cases.json")))


def case_tol(case):
    o = case.get("options", {})
    adam = o.get("optimizer", "SGD") != "SGD" or o.get("psi_optimizer", "SGD") != "SGD"
    return ADAM_TOL if adam else TOL


@pytest.mark.parametrize("name", sorted(CASES))
def test_gpu_matches_golden(name, built_library):
    case = CASES[name]
    ref = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    got = run_gpu(case)
    compare_outputs(ref, got, case_tol(case), name)


@pytest.mark.parametrize("name", ["dkp_tanh_small", "full_gelu_ce_adam", "simple_sigmoid_small"])
def test_gpu_without_graph_matches_golden(name, built_library):
    case = CASES[name]
    ref = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    compare_outputs(ref, run_gpu(case, use_graph=False), case_tol(case), name)


EXTRA = {
    # ragged everything: widths not multiples of 4, batch not a multiple of the tile
    "dkp_ragged": dict(kind="dkp", sizes=[13, 37, 37, 5, 3], batch=7, T=3, steps=2,
                       hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="sigmoid")),
    "dkp_single_weight_layer": dict(kind="dkp", sizes=[9, 4], batch=5, T=2, steps=2,
                                    hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "dkp_batch_one": dict(kind="dkp", sizes=[16, 16, 16, 4], batch=1, T=2, steps=2,
                          hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "dkp_wide_uniform": dict(kind="dkp", sizes=[64] + [128] * 6 + [10], batch=128, T=2, steps=2,
                             hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh")),
    "dkp_esigmoid_hardtanh": dict(kind="dkp", sizes=[20, 30, 30, 6], batch=10, T=2, steps=2,
                                  hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0,
                                             act="esigmoid")),
    "dkp_zero_steps": dict(kind="dkp", sizes=[20, 30, 30, 6], batch=10, T=0, steps=2,
                           hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="hard_tanh")),
    "simple_relu_ce": dict(kind="simple", sizes=[30, 40, 10], batch=16, T=5, steps=3,
                           hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="relu"),
                           options=dict(cross_entropy=1)),
    "full_plain": dict(kind="full", sizes=[30, 40, 40, 10], batch=16, T=4, steps=3,
                       hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="gelu")),
    "full_epc_residual": dict(kind="full", sizes=[30, 40, 40, 40, 10], batch=16, T=4, steps=3,
                              hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh"),
                              options=dict(epc=1, residual=1)),
    "full_epc_ce": dict(kind="full", sizes=[30, 40, 40, 10], batch=16, T=3, steps=2,
                        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="gelu"),
                        options=dict(epc=1, cross_entropy=1)),
    "full_adamw": dict(kind="full", sizes=[33, 40, 40, 10], batch=24, T=3, steps=3,
                       hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.01, act="tanh"),
                       options=dict(optimizer="ADAMW", psi_optimizer="ADAMW")),
}


@pytest.mark.parametrize("name", sorted(EXTRA))
def test_gpu_matches_live_oracle(name, built_library):
    case = EXTRA[name]
    compare_outputs(run_oracle(case), run_gpu(case), case_tol(case), name)


STAGED = ["dkp_ragged", "full_adamw", "full_epc_ce", "simple_relu_ce", "dkp_wide_uniform"]


@pytest.mark.parametrize("name", STAGED)
def test_staged_gradient_updates_match_oracle(name, built_library):
    """The stage / sum-over-shards / apply form of the weight updates (batch sharding) with one
    shard must give what the fused updates give."""
    case = EXTRA[name]
    compare_outputs(run_oracle(case), run_gpu(case, staged_gradients=True), case_tol(case), name)


def test_staged_gradients_ipc_and_center(built_library):
    case = dict(kind="full", sizes=[30, 40, 40, 10], batch=16, T=3, steps=2,
                hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="tanh"),
                options=dict(ipc=1, center_weights=1))
    compare_outputs(run_oracle(case), run_gpu(case, staged_gradients=True), TOL, "ipc staged")


# Shapes the tensor-core (tcgen05) kernels take: square layers, width a multiple of 256,
# batch a multiple of 128, with ordinary CUDA-core layers on both sides of the run.
TENSOR = {
    "dkp_tensor_run": dict(kind="dkp", sizes=[256] * 5 + [10], batch=128, T=2, steps=2,
                           hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "dkp_tensor_run_mixed": dict(kind="dkp", sizes=[100] + [512] * 4 + [10], batch=256, T=3,
                                 steps=2,
                                 hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="gelu")),
    # batch and width multiples of 256: the CTA-pair (cta_group::2) kernels
    "full_pair_tiles_residual_momentum": dict(
        kind="full", sizes=[64] + [256] * 4 + [10], batch=512, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="gelu"),
        options=dict(mupc=1, residual=1, momentum=0.9)),
    "full_tensor_run_residual_momentum": dict(
        kind="full", sizes=[64] + [256] * 4 + [10], batch=128, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="tanh"),
        options=dict(mupc=1, residual=1, momentum=0.9)),
}


def _tensor_run_of(case, precision):
    import ctypes
    from common import build_gpu_net
    from deepity_b200 import _lib
    net, _, _ = build_gpu_net(case, precision)
    lib = _lib.load()
    first, count = ctypes.c_int(), ctypes.c_int()
    lib.dpc_plan_tensor_run(lib.dpcn_plan(net._h), ctypes.byref(first), ctypes.byref(count))
    return first.value, count.value


@pytest.mark.parametrize("name", sorted(TENSOR))
def test_tensor_core_path_fp32_parity(name, built_library):
    """3xTF32 on the tensor cores is held to the same 1e-4 bound as the CUDA-core path."""
    case = TENSOR[name]
    assert _tensor_run_of(case, "fp32")[1] >= 3, "the tensor-core run was not detected"
    compare_outputs(run_oracle(case), run_gpu(case, precision="fp32"), TOL, name,
                    init=initial_parameters(case), delta_tol=DELTA_TOL)


@pytest.mark.parametrize("name", sorted(TENSOR))
def test_tensor_core_path_tf32_bound(name, built_library):
    """One TF32 pass: the reference's own 1e-2 CPU-vs-GPU bound."""
    case = TENSOR[name]
    compare_outputs(run_oracle(case), run_gpu(case, precision="tf32"), TF32_TOL, name,
                    init=initial_parameters(case), delta_tol=DELTA_TOL_TF32)


# Layers outside the run of identical square layers whose batch and output width are multiples of
# 256 (input width: any multiple of 8 from 64 up) run on the same CTA-pair tensor-core kernels, one
# launch per layer.
RECTANGULAR = {
    # 512->256 below and 256->512 above a run of two 256x256 layers, 512->10 on the CUDA cores
    "dkp_rectangular_around_run": dict(
        kind="dkp", sizes=[512, 256, 256, 256, 512, 10], batch=256, T=2, steps=2,
        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    # no two identical layers at all: rectangular layers only
    "dkp_rectangular_only": dict(
        kind="dkp", sizes=[256, 512, 256, 768, 10], batch=256, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="gelu")),
    # SimplePC layers (activation on the input side of the product) on the same kernels
    "simple_rectangular": dict(
        kind="simple", sizes=[256, 512, 256, 10], batch=256, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="tanh")),
    "simple_rectangular_decay_sigmoid": dict(
        kind="simple", sizes=[512, 256, 256, 10], batch=256, T=4, steps=2,
        hyper=dict(lr=0.01, ir=0.1, lmbda=0.01, act="sigmoid")),
    # the shape class of the wide benchmark network: wide input layer, softmax head, Adam.
    # (Adam's first steps move every element by about lr whatever its gradient, so an element
    # whose gradient is zero to rounding may move the other way: the rates keep twice that inside
    # the bound.)
    "full_wide_input_ce_adam": dict(
        kind="full", sizes=[768, 256, 256, 256, 10], batch=512, T=4, steps=3,
        hyper=dict(lr=1e-4, ir=0.1, fl=1e-4, lmbda=0.0, act="gelu"),
        options=dict(optimizer="ADAM", psi_optimizer="ADAM", cross_entropy=1)),
    # 784 inputs (not a multiple of the 32-wide K block nor of the 256-wide column tile): the last
    # K block of the forward product and the last column tile of the weight update are ragged
    "dkp_784_input": dict(
        kind="dkp", sizes=[784, 256, 256, 256, 10], batch=256, T=2, steps=2,
        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.01, act="tanh")),
    "full_784_input_ce_adam": dict(
        kind="full", sizes=[784, 512, 256, 10], batch=256, T=4, steps=3,
        hyper=dict(lr=1e-4, ir=0.1, fl=1e-4, lmbda=0.0, act="gelu"),
        options=dict(optimizer="ADAM", psi_optimizer="ADAM", cross_entropy=1)),
    "simple_784_input": dict(
        kind="simple", sizes=[784, 256, 256, 10], batch=256, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="tanh")),
    # a ragged width on a HIDDEN layer: its state update stops inside a column tile as well
    "dkp_ragged_hidden_width": dict(
        kind="dkp", sizes=[256, 264, 256, 10], batch=256, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh")),
    "simple_ragged_hidden_width": dict(
        kind="simple", sizes=[256, 328, 256, 10], batch=256, T=3, steps=2,
        hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="sigmoid")),
}
# which layer of a case the plan must report on the tensor cores (default: layer 0)
ON_TENSOR_CORES = {"dkp_ragged_hidden_width": "layer 1 (264->256)",
                   "simple_ragged_hidden_width": "layer 1 (328->256)"}


def _describe(case, precision):
    import ctypes
    from common import build_gpu_net
    from deepity_b200 import _lib
    net, _, _ = build_gpu_net(case, precision)
    lib = _lib.load()
    buf = ctypes.create_string_buffer(512)
    lib.dpc_plan_describe(lib.dpcn_plan(net._h), buf, 512)
    return buf.value.decode()


@pytest.mark.parametrize("name", sorted(RECTANGULAR))
@pytest.mark.parametrize("precision", ["fp32", "tf32"])
def test_rectangular_layers_on_tensor_cores(name, precision, built_library, monkeypatch):
    # (by default only layers of at least 2^29 multiply-adds per product leave the CUDA cores;
    # these small shapes are sent to the tensor cores to exercise every ragged edge)
    monkeypatch.setenv("DPC_RECTANGULAR_MIN_WORK", "0")
    case = RECTANGULAR[name]
    text = _describe(case, precision)
    first = case["sizes"][0], case["sizes"][1]
    want = ON_TENSOR_CORES.get(name, f"layer 0 ({first[0]}->{first[1]})")
    assert want in text or "layers 0.." in text, text
    adam = "optimizer" in case.get("options", {})
    tol = TF32_TOL if precision == "tf32" else (ADAM_TOL if adam else TOL)
    delta = DELTA_TOL_TF32 if precision == "tf32" else DELTA_TOL
    compare_outputs(run_oracle(case), run_gpu(case, precision=precision), tol, f"{name} {precision}",
                    init=None if adam else initial_parameters(case),
                    delta_tol=None if adam else delta)


def test_rectangular_layers_need_enough_work(built_library):
    """A single layer outside the run takes one launch per product: it goes to the tensor cores only
    when batch x inputs x outputs reaches 2^29 (below that the CUDA-core kernels, which take all
    layers of a phase in one launch, are as fast or faster)."""
    small = _describe(RECTANGULAR["simple_784_input"], "fp32")
    assert "on tcgen05" not in small, small
    big = dict(kind="full", sizes=[784, 1024, 1024, 10], batch=4096, T=2, steps=1,
               hyper=dict(lr=1e-4, ir=0.1, fl=1e-4, lmbda=0.0, act="gelu"),
               options=dict(optimizer="ADAM", psi_optimizer="ADAM", cross_entropy=1))
    text = _describe(big, "fp32")
    assert "layer 0 (784->1024) on tcgen05" in text, text


def test_simple_network_on_tensor_cores_by_default(built_library):
    """Four SimplePC layers of 2^29 multiply-adds each: on the tensor cores without any switch, the
    four launches of every phase side by side on the context's internal streams."""
    case = dict(kind="simple", sizes=[512] * 5 + [10], batch=2048, T=3, steps=2,
                hyper=dict(lr=0.01, ir=0.1, lmbda=0.0, act="tanh"))
    text = _describe(case, "fp32")
    assert "layer 0 (512->512) 1 (512->512) 2 (512->512) 3 (512->512) on tcgen05" in text, text
    compare_outputs(run_oracle(case), run_gpu(case, precision="fp32"), TOL, "simple, default path",
                    init=initial_parameters(case), delta_tol=DELTA_TOL)


def test_adam_on_tensor_core_layers(built_library):
    """Adam / AdamW weight updates of the tensor-core layers: product into the staging buffer,
    optimizer as an elementwise kernel; FullPC's decayed direct-feedback update on tensor cores."""
    case = dict(kind="full", sizes=[64] + [256] * 4 + [10], batch=256, T=3, steps=3,
                hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.01, act="gelu"),
                options=dict(optimizer="ADAMW", psi_optimizer="ADAM", cross_entropy=1))
    assert _tensor_run_of(case, "fp32")[1] >= 3
    ref = run_oracle(case)
    compare_outputs(ref, run_gpu(case, precision="fp32"), ADAM_TOL, "adam on tensor cores")


def test_mixed_precision_mode_bound(built_library):
    """precision="mixed": state path in 3xTF32, gradient path of the tensor-core layers in one
    TF32 pass (SGD only): held to 1e-3, and tighter than the all-TF32 mode."""
    case = dict(kind="dkp", sizes=[512] + [512] * 24 + [10], batch=1024, T=2, steps=3, seed=3,
                hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh"))
    ref = run_oracle(case)
    init = initial_parameters(case)
    mixed = compare_outputs(ref, run_gpu(case, precision="mixed"), 1e-3, "mixed", init=init,
                            delta_tol=DELTA_TOL_MIXED)
    tf32 = compare_outputs(ref, run_gpu(case, precision="tf32"), TF32_TOL, "tf32", init=init,
                           delta_tol=DELTA_TOL_TF32)
    assert mixed < tf32


def test_both_fp32_operand_splits(built_library, monkeypatch):
    """fp32 mode has two operand splits on the tensor cores: three BF16 passes (the default when
    every weight optimizer is SGD) and three TF32 passes (Adam-type networks, or on request).
    Both are held to the fp32 bound on the same SGD network; the TF32 split is the tighter one."""
    case = dict(kind="dkp", sizes=[512] + [512] * 12 + [10], batch=1024, T=2, steps=3, seed=5,
                hyper=dict(lr=1e-2, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh"))
    ref = run_oracle(case)
    init = initial_parameters(case)
    bf16 = compare_outputs(ref, run_gpu(case, precision="fp32"), TOL, "3xBF16 split", init=init,
                           delta_tol=DELTA_TOL)
    monkeypatch.setenv("DPC_FP32_SCHEME", "tf32x3")
    tf32 = compare_outputs(ref, run_gpu(case, precision="fp32"), TOL, "3xTF32 split", init=init,
                           delta_tol=DELTA_TOL)
    print(f"worst relative error: 3xBF16 {bf16:.2e}, 3xTF32 {tf32:.2e}")
    assert tf32 <= bf16


def test_deep_stack_at_benchmark_layer_shape(built_library):
    """48 layers of the deep-stack benchmark's shape (batch 1024, width 512): many tiles per
    CTA through the persistent pair kernels, the staged epilogue operands and the sequential
    sweep -- the place where a pipeline race would show."""
    case = dict(kind="dkp", sizes=[512] + [512] * 48 + [10], batch=1024, T=2, steps=2, seed=3,
                hyper=dict(lr=1e-3, ir=0.1, fl=1e-3, lmbda=0.0, act="tanh"))
    ref = run_oracle(case)
    init = initial_parameters(case)
    compare_outputs(ref, run_gpu(case, precision="fp32"), TOL, "deep stack fp32", init=init,
                    delta_tol=DELTA_TOL)
    compare_outputs(ref, run_gpu(case, precision="tf32"), TF32_TOL, "deep stack tf32", init=init,
                    delta_tol=DELTA_TOL_TF32)


def test_training_continues_to_track_the_oracle(built_library):
    """Ten consecutive steps: errors must not accumulate beyond the bound."""
    case = dict(kind="dkp", sizes=[32, 64, 64, 64, 10], batch=32, T=2, steps=10,
                hyper=dict(lr=0.01, ir=0.1, fl=0.01, lmbda=0.0, act="tanh"))
    compare_outputs(run_oracle(case), run_gpu(case), TOL, "ten steps")


def test_energy_decreases_over_training(built_library):
    # the sanity property of the reference's t*TrainStepSanity tests
    case = dict(kind="dkp", sizes=[32, 64, 64, 10], batch=32, T=2, steps=8,
                hyper=dict(lr=0.02, ir=0.1, fl=0.01, lmbda=0.0, act="tanh"))
    e = run_gpu(case)["energies"]
    assert np.all(np.isfinite(e)) and e[-1] < e[0]


def test_train_step_device_matches_host_entry(built_library):
    import torch
    from common import build_gpu_net
    case = CASES["dkp_tanh_small"]
    a, x, y = build_gpu_net(case)
    b, _, _ = build_gpu_net(case)
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    torch.cuda.synchronize()
    for _ in range(2):
        ea = a.train_step(x, y, case["T"])
        eb = b.train_step_device(xd, yd, case["T"])
        assert abs(ea - eb) <= 1e-6 * max(1.0, abs(ea))
    for l in range(len(case["sizes"]) - 1):
        assert np.array_equal(a.get_tensor(l, "W"), b.get_tensor(l, "W"))


def test_launch_counter_counts_graph_replays(built_library):
    from common import build_gpu_net
    net, x, y = build_gpu_net(CASES["dkp_tanh_small"])
    net.train_step(x, y, 2)
    n0 = net.launch_count
    net.train_step(x, y, 2)
    per_step = net.launch_count - n0
    assert per_step > 5
    net.train_step(x, y, 2)
    assert net.launch_count - n0 == 2 * per_step

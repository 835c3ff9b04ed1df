"""deepity_b200 — the predictive-coding train step of Deepity on NVIDIA B200 (sm_100a).

    from deepity_b200 import DKPPCN, Linear, TanH
    net = DKPPCN(Linear(784, 256), TanH(), Linear(256, 10), batch_size=256).configure(...)
    energy = net.train_step(x, y, inference_steps=2)

Everything computes in hand-written CUDA behind the C ABI of ``libdeepity_b200.so``
(``include/deepity_b200.h``); build it with ``python -m deepity_b200.build``.
"""
from .layer import (Activation, Convolution, ESigmoid, GeLU, HardTanH, Layer, Linear,  # noqa: F401
                    ReLU, Sigmoid, TanH)
from .networks import DKPPCN, FullPCN, SimplePCN  # noqa: F401
from .conv import SimpleConvolutionalPCN  # noqa: F401
from ._lib import DeepityError  # noqa: F401

__all__ = ["DKPPCN", "FullPCN", "SimplePCN", "SimpleConvolutionalPCN", "Convolution", "Linear", "Sigmoid", "TanH", "ReLU", "GeLU",
           "ESigmoid", "HardTanH", "DeepityError"]

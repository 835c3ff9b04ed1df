"""Architecture building blocks, same names and meaning as the reference's
``deepity/layer.py``: pass them positionally to a network's constructor."""
from __future__ import annotations


class Layer:
    def to_string(self) -> str:
        raise NotImplementedError


class Linear(Layer):
    """A weighted layer of shape (in_n, out_n)."""

    def __init__(self, in_n: int, out_n: int):
        self.in_n = int(in_n)
        self.out_n = int(out_n)

    def to_string(self) -> str:
        return "linear"


class Convolution(Layer):
    """A 2-D convolutional layer (``deepity/layer.py:26-48``); ``out_channels = 0`` closes the
    architecture with the terminal layer, which has no weights."""

    def __init__(self, out_channels: int, kernel_h: int, kernel_w: int, stride_h: int = 1,
                 stride_w: int = 1, pad_h: int = 0, pad_w: int = 0):
        self.out_channels = int(out_channels)
        self.kernel_h, self.kernel_w = int(kernel_h), int(kernel_w)
        self.stride_h, self.stride_w = int(stride_h), int(stride_w)
        self.pad_h, self.pad_w = int(pad_h), int(pad_w)

    def to_string(self) -> str:
        return "convolution"


class Activation:
    def to_string(self) -> str:
        raise NotImplementedError


class Sigmoid(Activation):
    """Logistic sigmoid activation."""

    def to_string(self) -> str:
        return "sigmoid"


class TanH(Activation):
    """Hyperbolic tangent activation."""

    def to_string(self) -> str:
        return "tanh"


class ReLU(Activation):
    """Rectified linear unit activation."""

    def to_string(self) -> str:
        return "relu"


class GeLU(Activation):
    """Gaussian error linear unit activation (tanh approximation)."""

    def to_string(self) -> str:
        return "gelu"


class ESigmoid(Activation):
    """Rational 'elliot' sigmoid 0.5 + 0.5 z/(1+|z|)."""

    def to_string(self) -> str:
        return "esigmoid"


class HardTanH(Activation):
    """clamp(z, -1, 1)."""

    def to_string(self) -> str:
        return "hard_tanh"


# name -> dpc_act id (the forward enumerators of the reference's ActivationType).
ACT_IDS = {"relu": 0, "gelu": 2, "sigmoid": 4, "esigmoid": 6, "tanh": 8, "linear": 10,
           "hard_tanh": 12}
OPT_IDS = {"SGD": 0, "ADAM": 1, "ADAMW": 2}

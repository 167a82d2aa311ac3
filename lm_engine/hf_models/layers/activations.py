"""Activation registry: plain activations by name and gated (``*glu``) variants.

Parity: lm_engine/hf_models/modeling_utils/activations/{base,glu,__init__}.py. A gated activation consumes a
projection of width 2I laid out as ``[up | gate]`` and returns ``up * act(gate)``; ``swiglu`` runs the fused kernel.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...enums import Kernel
from ...kernels import is_kernel_allowed, wait_for_ACT


class _Lambda(nn.Module):
    def __init__(self, fn) -> None:
        super().__init__()
        self.fn = fn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fn(x)


def _gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


def _quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


def _gelu_fast(x):
    return 0.5 * x * (1.0 + torch.tanh(x * 0.7978845608 * (1.0 + 0.044715 * x * x)))


def _laplace(x, mu=0.707107, sigma=0.282095):
    return 0.5 * (1.0 + torch.erf((x - mu) / (sigma * math.sqrt(2.0))))


def _relu_squared(x):
    return torch.square(F.relu(x))


_BASE = {
    "celu": nn.CELU, "elu": nn.ELU, "gelu": nn.GELU, "hard_shrink": nn.Hardshrink, "hard_sigmoid": nn.Hardsigmoid,
    "hard_swish": nn.Hardswish, "hard_tanh": nn.Hardtanh, "identity": nn.Identity, "leaky_reLU": nn.LeakyReLU,
    "log_sigmoid": nn.LogSigmoid, "mish": nn.Mish, "prelu": nn.PReLU, "relu": nn.ReLU, "relu6": nn.ReLU6,
    "rrelu": nn.RReLU, "sigmoid": nn.Sigmoid, "selu": nn.SELU, "silu": nn.SiLU, "swish": nn.SiLU,
    "softplus": nn.Softplus, "soft_plus": nn.Softplus, "soft_shrink": nn.Softshrink, "soft_sign": nn.Softsign,
    "tanh": nn.Tanh, "tanh_shrink": nn.Tanhshrink,
}
_FUNCTIONAL = {
    "gelu_pytorch_tanh": _gelu_tanh, "gelu_new": _gelu_tanh, "gelu_fast": _gelu_fast, "quick_gelu": _quick_gelu,
    "gelu_10": lambda x: torch.clamp(F.gelu(x), -10, 10), "laplace": _laplace, "relu2": _relu_squared,
    "relu_squared": _relu_squared, "linear": lambda x: x,
}
# gated name -> name of the activation applied to the gate half
_GLU = {
    "bilinear": "identity", "ceglu": "celu", "eglu": "elu", "geglu": "gelu", "glu": "sigmoid", "miglu": "mish",
    "mishglu": "mish", "preglu": "prelu", "reglu": "relu", "rreglu": "rrelu", "seglu": "selu", "swiglu": "swish",
}


def is_glu(name: str) -> bool:
    return name.endswith("glu")


def get_base_activation(name: str) -> nn.Module:
    if name in _BASE:
        return _BASE[name]()
    if name in _FUNCTIONAL:
        return _Lambda(_FUNCTIONAL[name])
    raise ValueError(f"invalid activation function ({name})")


class GLUActivation(nn.Module):
    def __init__(self, base: nn.Module, fused_swiglu: bool = False) -> None:
        super().__init__()
        self.base = base
        self.fused_swiglu = fused_swiglu

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused_swiglu and is_kernel_allowed(Kernel.swiglu_packed_cute):
            x = wait_for_ACT(x, wait_in_forward=True, wait_in_backward=False)
            x = ops.swiglu_packed(x)
            return wait_for_ACT(x, wait_in_forward=False, wait_in_backward=True)
        up, gate = x.chunk(2, dim=-1)
        return up * self.base(gate)


def get_glu_activation(name: str) -> nn.Module:
    if name in ("glu", "sigmoid_glu"):
        base = nn.Sigmoid()
    elif name in _GLU:
        base = get_base_activation(_GLU[name])
    elif name.endswith("_glu"):
        base = get_base_activation(name[: -len("_glu")])
    else:
        raise ValueError(f"invalid activation function ({name})")
    return GLUActivation(base, fused_swiglu=name in ("swiglu", "swish_glu", "silu_glu"))


def get_activation_function(name: str) -> nn.Module:
    return get_glu_activation(name) if is_glu(name) else get_base_activation(name)

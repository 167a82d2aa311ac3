"""Normalisation layers (parity: lm_engine/hf_models/modeling_utils/normalization.py:19-72). All norm parameters
are excluded from weight decay; RMSNorm runs the fused kernel when ``rmsnorm_cute`` is enabled."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...enums import Kernel
from ...kernels import is_kernel_allowed, wait_for_ACT
from ..parameter import mark_parameter_as_no_weight_decay


class LayerNorm(nn.LayerNorm):
    def __init__(self, normalized_shape: int, eps: float = 1e-6) -> None:
        super().__init__(normalized_shape, eps=eps)
        mark_parameter_as_no_weight_decay(self.weight)
        mark_parameter_as_no_weight_decay(self.bias)


class RMSNorm(nn.RMSNorm):
    def __init__(self, normalized_shape: int, eps: float = 1e-6) -> None:
        super().__init__(normalized_shape, eps=eps)
        mark_parameter_as_no_weight_decay(self.weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if is_kernel_allowed(Kernel.rmsnorm_cute) or is_kernel_allowed(Kernel.rmsnorm_memory_efficient_cute):
            x = wait_for_ACT(x, wait_in_forward=True, wait_in_backward=False)
            x = ops.rmsnorm(x, self.weight, self.eps)
            return wait_for_ACT(x, wait_in_forward=False, wait_in_backward=True)
        return super().forward(x)


class SiluGatedRMSNorm(RMSNorm):
    """``rmsnorm(x * silu(gate))`` evaluated in fp32 (used by the Mamba-2 mixer)."""

    def forward(self, x: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
        dtype = x.dtype
        x = x.float()
        if gate is not None:
            x = x * F.silu(gate.float())
        x = F.rms_norm(x, self.normalized_shape, None if self.weight is None else self.weight.float(), self.eps)
        return x.to(dtype)


_NORMS = {"layernorm": LayerNorm, "rmsnorm": RMSNorm, "silu_gated_rmsnorm": SiluGatedRMSNorm}


def get_normalization_function(name: str | None, normalized_shape: int, eps: float = 1e-5) -> nn.Module:
    if name is None:
        return nn.Identity()
    if name not in _NORMS:
        raise ValueError(f"unexpected `normalization_function` {name}")
    return _NORMS[name](normalized_shape, eps=eps)

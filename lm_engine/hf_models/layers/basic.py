"""Linear / embedding / conv modules that carry their init std (parity: lm_engine/hf_models/modeling_utils/linear.py,
embedding.py, convolution.py). Weights ~ N(0, std), biases zero and excluded from weight decay. The linear and
embedding forward passes go through :mod:`lm_engine.ops` (tcgen05 GEMM / gather kernels on sm_100a)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ..parameter import mark_parameter_as_no_weight_decay


def loaded_from_checkpoint(p: torch.Tensor) -> bool:
    """True for a tensor that ``from_pretrained`` already filled; initialisers must leave it alone (the loader only
    guards the ``torch.nn.init`` functions, not plain in-place writes)."""
    return getattr(p, "_is_hf_initialized", False)


def init_zeros_(p: torch.Tensor | None) -> None:
    if p is not None and not loaded_from_checkpoint(p):
        p.zero_()


def init_fill_(p: torch.Tensor | None, value) -> None:
    if p is not None and not loaded_from_checkpoint(p):
        if torch.is_tensor(value):
            p.copy_(value)
        else:
            p.fill_(value)


class ParameterizedLinear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 std: float | None = None) -> None:
        self.std = std
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        mark_parameter_as_no_weight_decay(self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.std is None:
            super().reset_parameters()
        else:
            nn.init.normal_(self.weight, mean=0.0, std=self.std)
        init_zeros_(getattr(self, "bias", None))


class ParameterizedEmbedding(nn.Embedding):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None, device=None,
                 dtype=None, std: float | None = None) -> None:
        self.std = std
        super().__init__(num_embeddings, embedding_dim, padding_idx=padding_idx, device=device, dtype=dtype)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(self.weight, ids)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.std is None:
            super().reset_parameters()
        else:
            nn.init.normal_(self.weight, mean=0.0, std=self.std)
            if self.padding_idx is not None and not loaded_from_checkpoint(self.weight):
                self.weight[self.padding_idx].zero_()


class ParameterizedConv1d(nn.Conv1d):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, padding: int = 0,
                 dilation: int = 1, groups: int = 1, bias: bool = True, padding_mode: str = "zeros", device=None,
                 dtype=None, std: float | None = None) -> None:
        self.std = std
        super().__init__(in_channels, out_channels, kernel_size, stride=stride, padding=padding, dilation=dilation,
                         groups=groups, bias=bias, padding_mode=padding_mode, device=device, dtype=dtype)
        mark_parameter_as_no_weight_decay(self.bias)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.std is None:
            super().reset_parameters()
        else:
            nn.init.normal_(self.weight, mean=0.0, std=self.std)
            init_zeros_(getattr(self, "bias", None))


def dropout(p: float) -> nn.Module:
    return nn.Identity() if p == 0 else nn.Dropout(p)

"""Causal convolution mixer: linear -> grouped causal conv1d -> activation (gated variants allowed) -> linear
(parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/causal_convolution.py:37-229). During decoding the
last ``kernel_size - 1`` inputs are the cached state."""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..context import SequenceContext
from ..parameter import mark_parameter_as_mup_learning_rate
from .activations import get_activation_function, is_glu
from .basic import ParameterizedConv1d, ParameterizedLinear


def causal_conv1d_torch(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, groups: int,
                        state: torch.Tensor | None = None) -> torch.Tensor:
    """x ``[b, c_in, s]``; left-pads with ``state`` (``[b, c_in, k-1]``) or zeros so that output t sees inputs <= t."""
    k = weight.shape[-1]
    pad = state if state is not None else x.new_zeros(x.shape[0], x.shape[1], k - 1)
    return F.conv1d(torch.cat([pad, x], dim=-1), weight, bias, groups=groups)


class CausalConvolution(nn.Module):
    def __init__(self, hidden_size: int, in_channels: int, out_channels: int, kernel_size: int, num_groups: int,
                 activation_function: str, add_bias: bool, init_method: str, initializer_range: float,
                 m_width: float | None, num_layers: int, layer_idx: int | None, use_padding_free_transformer: bool) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.kernel_size = kernel_size
        self.num_groups = num_groups
        self.in_channels = in_channels
        self.use_padding_free_transformer = use_padding_free_transformer
        gated = is_glu(activation_function)
        std = initializer_range / (math.sqrt(m_width) if init_method == "mup" else 1)
        self.input_projection = ParameterizedLinear(hidden_size, in_channels, bias=add_bias, std=std)
        self.conv1d = ParameterizedConv1d(in_channels, out_channels, kernel_size, groups=num_groups, bias=add_bias, std=std)
        self.activation_function = get_activation_function(activation_function)
        out_std = std / math.sqrt(2 * num_layers)
        self.output_projection = ParameterizedLinear(out_channels // 2 if gated else out_channels, hidden_size, bias=False, std=out_std)
        for m in (self.input_projection, self.conv1d, self.output_projection):
            mark_parameter_as_mup_learning_rate(m.weight)

    def _conv(self, x: torch.Tensor, state: torch.Tensor | None) -> torch.Tensor:
        return causal_conv1d_torch(x, self.conv1d.weight, self.conv1d.bias, self.num_groups, state)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        x = self.input_projection(hidden_states)
        depthwise = self.num_groups == self.in_channels == self.conv1d.out_channels
        if ctx.packed and depthwise and x.is_cuda:
            from ...ops.sequence import causal_conv1d_packed

            y = causal_conv1d_packed(x, self.conv1d.weight, self.conv1d.bias, ctx.cu_seqlens)  # no host round trip
        elif ctx.packed:
            bounds = ctx.cu_seqlens.tolist()
            pieces = [self._conv(x[s:e].t().unsqueeze(0), None).squeeze(0).t() for s, e in zip(bounds[:-1], bounds[1:]) if e > s]
            y = torch.cat(pieces, dim=0)
        else:
            if ctx.attention_mask is not None and past_key_values is None:
                x = x * ctx.attention_mask[:, -x.shape[1]:, None].to(x.dtype)
            xc = x.transpose(1, 2)
            state = None if past_key_values is None else past_key_values.get_cache(self.layer_idx)
            y = self._conv(xc, state).transpose(1, 2)
            if past_key_values is not None:
                history = xc if state is None else torch.cat([state, xc], dim=-1)
                window = history[..., -(self.kernel_size - 1):] if self.kernel_size > 1 else history[..., :0]
                if window.shape[-1] < self.kernel_size - 1:
                    window = F.pad(window, (self.kernel_size - 1 - window.shape[-1], 0))
                past_key_values.update(state=window, num_tokens_added=x.shape[1], layer_idx=self.layer_idx)
        return self.output_projection(self.activation_function(y))

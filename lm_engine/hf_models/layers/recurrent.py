"""Multi-head recurrent mixers with block-diagonal state transitions: a plain tanh RNN and a GRU
(parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/{rnn.py:25-151, gru.py:25-160}).

Per head ``n`` with state width ``d`` (``state_weight[n]`` is ``[d, d]``):
    RNN:  h_t = tanh(h_{t-1} W + x_t)
    GRU:  f = sigmoid(h W_f + x_f),  r = sigmoid(h W_r + x_r),  z = tanh((r * h) W + x),  h_t = f * h + (1 - f) * z
Inputs and weights are scaled by ``1 / sqrt(input_size + d)``. ``gradient_clipping`` clamps the gradient that flows
back through the state at every step. Packed batches run one scan per document; padded batches zero the
contribution of masked positions.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ...utils import divide_if_divisible
from ..context import SequenceContext
from ..parameter import mark_parameter_as_mup_learning_rate, mark_parameter_as_no_weight_decay
from .basic import ParameterizedLinear
from .normalization import get_normalization_function


class _ClipGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, limit):
        ctx.limit = limit
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad.clamp(-ctx.limit, ctx.limit), None


def _clip(x: torch.Tensor, limit: float | None) -> torch.Tensor:
    return x if limit is None else _ClipGradient.apply(x, limit)


def rnn_scan(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, clip: float | None) -> torch.Tensor:
    """x ``[b, s, n, d]``, weight ``[n, d, d]`` -> all states ``[b, s, n, d]``."""
    b, s, n, d = x.shape
    h = x.new_zeros(b, n, d) if state is None else state
    out = []
    for t in range(s):
        h = _clip(h, clip)
        h = torch.tanh(torch.einsum("bnd,nde->bne", h, weight) + x[:, t])
        out.append(h)
    return torch.stack(out, dim=1)


def gru_scan(x, weight, fx, f_weight, rx, r_weight, state, clip) -> torch.Tensor:
    b, s, n, d = x.shape
    h = x.new_zeros(b, n, d) if state is None else state
    out = []
    for t in range(s):
        h = _clip(h, clip)
        f = torch.sigmoid(torch.einsum("bnd,nde->bne", h, f_weight) + fx[:, t])
        r = torch.sigmoid(torch.einsum("bnd,nde->bne", h, r_weight) + rx[:, t])
        z = torch.tanh(torch.einsum("bnd,nde->bne", r * h, weight) + x[:, t])
        h = f * h + (1 - f) * z
        out.append(h)
    return torch.stack(out, dim=1)


class _RecurrentBase(nn.Module):
    gates = 1

    def __init__(self, input_size: int, state_size: int, output_size: int, num_heads: int, add_bias: bool,
                 gradient_clipping: float | None, initializer_range: float, m_width: float | None, init_method: str,
                 normalization_function: str | None, num_layers: int, layer_idx: int | None,
                 use_padding_free_transformer: bool, layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        self.input_size, self.state_size, self.output_size = input_size, state_size, output_size
        self.num_heads = num_heads
        self.gradient_clipping = gradient_clipping
        self.layer_idx = layer_idx
        self.use_padding_free_transformer = use_padding_free_transformer
        self.state_head_dim = divide_if_divisible(state_size, num_heads, "state_size must be divisible by num_heads")
        self.is_gated_normalization = normalization_function == "silu_gated_rmsnorm"
        std = initializer_range / (math.sqrt(m_width) if init_method == "mup" else 1)
        self.state_weight_std = std
        width = self.gates * state_size + (state_size if self.is_gated_normalization else 0)
        self.input_projection = ParameterizedLinear(input_size, width, bias=add_bias, std=std)
        self.state_weight = nn.Parameter(torch.empty(self.gates * num_heads, self.state_head_dim, self.state_head_dim))
        out_std = initializer_range / math.sqrt(2 * num_layers) / (math.sqrt(m_width) if init_method == "mup" else 1)
        self.output_projection = ParameterizedLinear(state_size, output_size, bias=False, std=out_std)
        self.norm = get_normalization_function(normalization_function, state_size, eps=layer_norm_epsilon)
        self.factor = 1 / math.sqrt(input_size + self.state_head_dim)
        self.reset_parameters()
        mark_parameter_as_mup_learning_rate(self.input_projection.weight)
        mark_parameter_as_mup_learning_rate(self.state_weight)
        mark_parameter_as_mup_learning_rate(self.output_projection.weight)
        mark_parameter_as_no_weight_decay(self.state_weight)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.state_weight, std=self.state_weight_std)

    def _scan(self, x: torch.Tensor, state: torch.Tensor | None) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        x = self.input_projection(hidden_states)
        gate = None
        if self.is_gated_normalization:
            x, gate = x.split((self.gates * self.state_size, self.state_size), dim=-1)
        x = x * self.factor
        if ctx.packed:
            bounds = ctx.cu_seqlens.tolist()
            pieces = [self._scan(x[s:e].unsqueeze(0), None).squeeze(0) for s, e in zip(bounds[:-1], bounds[1:]) if e > s]
            h = torch.cat(pieces, dim=0)
        else:
            if ctx.attention_mask is not None and past_key_values is None and not bool(torch.all(ctx.attention_mask == 1)):
                # left padding: a zero input keeps tanh(0) = 0 state contributions out of real positions
                x = x * ctx.attention_mask[:, -x.shape[1]:, None].to(x.dtype)
            state = None if past_key_values is None else past_key_values.get_cache(self.layer_idx)
            h = self._scan(x, state)
            if past_key_values is not None:
                past_key_values.update(state=h[:, -1].reshape(h.shape[0], self.num_heads, self.state_head_dim),
                                       num_tokens_added=x.shape[1], layer_idx=self.layer_idx)
        h = h.reshape(*h.shape[:-2], self.state_size)
        h = self.norm(h, gate) if self.is_gated_normalization else self.norm(h)
        return self.output_projection(h)

    def extra_repr(self) -> str:
        return f"gradient_clipping = {self.gradient_clipping}\nweight_shape: {tuple(self.state_weight.shape)}"


class RNN(_RecurrentBase):
    gates = 1

    def _scan(self, x, state):
        x = x.reshape(*x.shape[:-1], self.num_heads, self.state_head_dim)
        return rnn_scan(x, self.state_weight * self.factor, state, self.gradient_clipping)


class GRU(_RecurrentBase):
    gates = 3

    def _scan(self, x, state):
        xi, xf, xr = (t.reshape(*t.shape[:-1], self.num_heads, self.state_head_dim) for t in x.chunk(3, dim=-1))
        w, wf, wr = (self.state_weight * self.factor).chunk(3, dim=0)
        return gru_scan(xi, w, xf, wf, xr, wr, state, self.gradient_clipping)

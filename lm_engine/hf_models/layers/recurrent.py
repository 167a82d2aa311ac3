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

from ...enums import Kernel
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

    kernel_name = None  # the switch that turns on the native scan for this mixer

    def _kernel_ok(self, x: torch.Tensor) -> bool:
        from ...kernels import is_kernel_allowed
        from ...ops.recurrent import recurrent_kernel_ok

        return is_kernel_allowed(self.kernel_name) and recurrent_kernel_ok(x, self.state_head_dim)

    def _masked_input_and_state(self, x: torch.Tensor, ctx: SequenceContext, past_key_values):
        if ctx.attention_mask is not None and past_key_values is None and not bool(torch.all(ctx.attention_mask == 1)):
            # left padding: a zero input keeps tanh(0) = 0 state contributions out of real positions
            x = x * ctx.attention_mask[:, -x.shape[1]:, None].to(x.dtype)
        state = None if past_key_values is None else past_key_values.get_cache(self.layer_idx)
        return x, state

    def _store_state(self, h: torch.Tensor, num_tokens: int, past_key_values) -> None:
        if past_key_values is not None:
            past_key_values.update(state=h[:, -1].reshape(h.shape[0], self.num_heads, self.state_head_dim),
                                   num_tokens_added=num_tokens, layer_idx=self.layer_idx)

    def _native_scan(self, x: torch.Tensor, ctx: SequenceContext, past_key_values) -> torch.Tensor:
        """The scan kernel over the packed token rows (a padded batch is ``batch`` documents of equal length)."""
        from ...ops.recurrent import recurrent_scan

        weight = self.state_weight * self.factor
        gru = self.gates == 3
        if ctx.packed:
            return recurrent_scan(x, weight, ctx.cu_seqlens_int32(), self.num_heads, self.state_head_dim, gru, self.gradient_clipping)
        x, state = self._masked_input_and_state(x, ctx, past_key_values)
        b, s, width = x.shape
        cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32, device=x.device)
        h = recurrent_scan(x.reshape(b * s, width), weight, cu, self.num_heads, self.state_head_dim, gru, self.gradient_clipping, h0=state)
        h = h.view(b, s, self.num_heads, self.state_head_dim)
        self._store_state(h, s, past_key_values)
        return h

    def _scan(self, x: torch.Tensor, state: torch.Tensor | None) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        x = self.input_projection(hidden_states)
        gate = None
        if self.is_gated_normalization:
            x, gate = x.split((self.gates * self.state_size, self.state_size), dim=-1)
        x = x * self.factor
        if self._kernel_ok(x):
            h = self._native_scan(x, ctx, past_key_values)
        elif ctx.packed:
            bounds = ctx.cu_seqlens.tolist()
            pieces = [self._scan(x[s:e].unsqueeze(0), None).squeeze(0) for s, e in zip(bounds[:-1], bounds[1:]) if e > s]
            h = torch.cat(pieces, dim=0)
        else:
            x, state = self._masked_input_and_state(x, ctx, past_key_values)
            h = self._scan(x, state)
            self._store_state(h, x.shape[1], past_key_values)
        h = h.reshape(*h.shape[:-2], self.state_size)
        h = self.norm(h, gate) if self.is_gated_normalization else self.norm(h)
        return self.output_projection(h)

    def extra_repr(self) -> str:
        return f"gradient_clipping = {self.gradient_clipping}\nweight_shape: {tuple(self.state_weight.shape)}"


class RNN(_RecurrentBase):
    gates = 1
    kernel_name = Kernel.rnn_cute

    def _scan(self, x, state):
        x = x.reshape(*x.shape[:-1], self.num_heads, self.state_head_dim)
        return rnn_scan(x, self.state_weight * self.factor, state, self.gradient_clipping)


class GRU(_RecurrentBase):
    gates = 3
    kernel_name = Kernel.gru_cute

    def _scan(self, x, state):
        xi, xf, xr = (t.reshape(*t.shape[:-1], self.num_heads, self.state_head_dim) for t in x.chunk(3, dim=-1))
        w, wf, wr = (self.state_weight * self.factor).chunk(3, dim=0)
        return gru_scan(xi, w, xf, wf, xr, wr, state, self.gradient_clipping)

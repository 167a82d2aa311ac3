"""Mamba-2 mixer (state space duality, arXiv 2405.21060) in plain PyTorch.

Parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/mamba2.py:85-575 (parameter names ``in_proj``,
``conv1d``, ``dt_bias``, ``A_log``, ``D``, ``norm``, ``out_proj``; ``A_log = log(1..H)``, ``D = dt_bias = 1``).
``in_proj`` yields (gate, xBC, dt); xBC goes through a depthwise causal convolution and an activation and splits into
x, B, C; the selective scan runs chunk-wise (quadratic inside a chunk, a linear recurrence over chunk states); the
result is gated-RMS-normalised and projected out. Decoding updates a (conv window, ssm state) cache one token at a time.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...utils import divide_if_divisible
from ..context import SequenceContext
from ..parameter import mark_parameter_as_mup_learning_rate, mark_parameter_as_no_weight_decay
from .activations import get_activation_function
from .basic import ParameterizedConv1d, ParameterizedLinear, init_fill_
from .normalization import get_normalization_function


def _segment_sums(a: torch.Tensor) -> torch.Tensor:
    """``out[..., i, j] = sum_{j < k <= i} a[..., k]`` for ``j <= i`` and ``-inf`` above the diagonal."""
    n = a.shape[-1]
    c = a.cumsum(-1)
    diff = c[..., :, None] - c[..., None, :]
    keep = torch.ones(n, n, dtype=torch.bool, device=a.device).tril()
    return diff.masked_fill(~keep, float("-inf"))


def ssd_chunk_scan(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, chunk: int,
                   initial_state: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """x ``[B, L, H, P]`` (already multiplied by dt), a ``[B, L, H]`` (= A * dt), b / c ``[B, L, H, N]``.
    Returns ``(y [B, L, H, P], final_state [B, H, P, N])``."""
    B_, L, H, P = x.shape
    pad = (chunk - L % chunk) % chunk
    if pad:
        x, a, b, c = (F.pad(t, (0, 0) * (t.dim() - 2) + (0, pad)) for t in (x, a, b, c))
    nc = x.shape[1] // chunk
    x, b, c = (t.reshape(B_, nc, chunk, *t.shape[2:]) for t in (x, b, c))
    a = a.reshape(B_, nc, chunk, H).permute(0, 3, 1, 2)  # [B, H, nc, chunk]
    a_cum = a.cumsum(-1)

    within = torch.exp(_segment_sums(a))  # [B, H, nc, chunk, chunk]
    y_diag = torch.einsum("bclhn,bcshn,bhcls,bcshp->bclhp", c, b, within, x)

    decay_to_end = torch.exp(a_cum[..., -1:] - a_cum)
    states = torch.einsum("bclhn,bhcl,bclhp->bchpn", b, decay_to_end, x)
    if initial_state is None:
        initial_state = states.new_zeros(B_, 1, H, P, states.shape[-1])
    else:
        initial_state = initial_state.unsqueeze(1)
    states = torch.cat([initial_state, states], dim=1)
    chunk_decay = torch.exp(_segment_sums(F.pad(a_cum[..., -1], (1, 0))))  # [B, H, nc + 1, nc + 1]
    carried = torch.einsum("bhzc,bchpn->bzhpn", chunk_decay, states)
    entering, final_state = carried[:, :-1], carried[:, -1]

    y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", c, entering, torch.exp(a_cum))
    y = (y_diag + y_off).reshape(B_, nc * chunk, H, P)
    return y[:, :L], final_state


class Mamba2(nn.Module):
    def __init__(self, hidden_size: int, ssm_state_size: int, ssm_intermediate_size: int, ssm_num_heads: int,
                 conv_kernel_size: int, time_step_limit: tuple[float, float], add_bias: bool, use_conv_bias: bool,
                 ssm_activation_function: str, num_groups: int, chunk_size: int, layer_norm_epsilon: float,
                 initializer_range: float, m_width: float | None, init_method: str, num_layers: int, layer_idx: int | None) -> None:
        super().__init__()
        self.num_heads = ssm_num_heads
        self.hidden_size = hidden_size
        self.ssm_state_size = ssm_state_size
        self.conv_kernel_size = conv_kernel_size
        self.intermediate_size = ssm_intermediate_size
        self.layer_idx = layer_idx
        self.n_groups = num_groups
        self.head_dim = divide_if_divisible(ssm_intermediate_size, ssm_num_heads, "")
        self.chunk_size = chunk_size
        self.time_step_limit = tuple(time_step_limit)
        self.activation = get_activation_function(ssm_activation_function)
        self._silu_activation = ssm_activation_function in ("silu", "swish")

        std = initializer_range / (math.sqrt(m_width) if init_method == "mup" else 1)
        self.conv_dim = self.intermediate_size + 2 * self.n_groups * self.ssm_state_size
        self.conv1d = ParameterizedConv1d(self.conv_dim, self.conv_dim, conv_kernel_size, groups=self.conv_dim,
                                          padding=conv_kernel_size - 1, bias=use_conv_bias, std=std)
        self.in_proj = ParameterizedLinear(hidden_size, self.intermediate_size + self.conv_dim + self.num_heads, bias=add_bias, std=std)
        self.dt_bias = nn.Parameter(torch.ones(self.num_heads))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, self.num_heads + 1, dtype=torch.float32)))
        self.norm = get_normalization_function("silu_gated_rmsnorm", self.intermediate_size, eps=layer_norm_epsilon)
        self.D = nn.Parameter(torch.ones(self.num_heads))
        self.out_proj = ParameterizedLinear(self.intermediate_size, hidden_size, bias=add_bias, std=std / math.sqrt(2 * num_layers))
        for p in (self.dt_bias, self.A_log, self.D):
            mark_parameter_as_no_weight_decay(p)
        for p in (self.A_log, self.D, self.conv1d.weight, self.in_proj.weight, self.out_proj.weight):
            mark_parameter_as_mup_learning_rate(p)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        init_fill_(self.A_log, torch.log(torch.arange(1, self.num_heads + 1, dtype=torch.float32)))
        init_fill_(self.D, 1.0)
        init_fill_(self.dt_bias, 1.0)

    def _split(self, projected: torch.Tensor):
        return projected.split([self.intermediate_size, self.conv_dim, self.num_heads], dim=-1)

    def _scan_kernel_ok(self, xbc: torch.Tensor) -> bool:
        from ...enums import Kernel
        from ...kernels import is_kernel_allowed
        from ...ops.ssd import ssd_kernel_ok

        return is_kernel_allowed(Kernel.mamba2_ssm) and ssd_kernel_ok(xbc.new_empty(0, self.head_dim), self.ssm_state_size)

    def _ssm_inputs(self, xbc: torch.Tensor, dt: torch.Tensor, repeat_groups: bool = True):
        gn = self.n_groups * self.ssm_state_size
        x, b, c = xbc.split([self.intermediate_size, gn, gn], dim=-1)
        lead = x.shape[:-1]
        x = x.reshape(*lead, self.num_heads, self.head_dim)
        rep = self.num_heads // self.n_groups if repeat_groups else 1
        b = b.reshape(*lead, self.n_groups, self.ssm_state_size).repeat_interleave(rep, dim=-2)
        c = c.reshape(*lead, self.n_groups, self.ssm_state_size).repeat_interleave(rep, dim=-2)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        lo, hi = self.time_step_limit
        if lo > 0 or hi != float("inf"):
            dt = dt.clamp(lo, hi)
        return x, b, c, dt

    def _sequence(self, u: torch.Tensor, mask: torch.Tensor | None, cache, cu_seqlens: torch.Tensor | None = None) -> torch.Tensor:
        """u ``[B, L, hidden]``; with ``cu_seqlens`` (kernels only) the single row holds packed documents."""
        dtype = u.dtype
        gate, xbc, dt = self._split(self.in_proj(u))
        if mask is not None:
            xbc = xbc * mask[..., None].to(xbc.dtype)
        conv_in = xbc.transpose(1, 2)
        if xbc.is_cuda and self._silu_activation and self.conv_kernel_size <= 8:
            from ...ops.sequence import causal_conv1d_packed

            # every row of the batch is one sequence: depthwise conv + SiLU in one kernel on the [tokens, channels] layout
            rows, length = xbc.shape[:2]
            cu = cu_seqlens if cu_seqlens is not None else torch.arange(0, rows * length + 1, length, dtype=torch.int32, device=xbc.device)
            xbc_act = causal_conv1d_packed(xbc.reshape(rows * length, -1), self.conv1d.weight, self.conv1d.bias, cu, "silu").view_as(xbc)
        else:
            conv_out = self.conv1d(conv_in)[..., : conv_in.shape[-1]]
            xbc_act = self.activation(conv_out.transpose(1, 2))
        if mask is not None:
            xbc_act = xbc_act * mask[..., None].to(xbc_act.dtype)
        A = -torch.exp(self.A_log.float())
        if self._scan_kernel_ok(xbc_act):
            from ...ops.ssd import ssd_scan

            # b and c stay per group: the scan kernel maps heads to groups itself
            x, b, c, dt = self._ssm_inputs(xbc_act, dt, repeat_groups=False)
            y, final_state = ssd_scan(x.float() * dt[..., None], A * dt, b, c, cu_seqlens=cu_seqlens)
        else:
            x, b, c, dt = self._ssm_inputs(xbc_act, dt)
            y, final_state = ssd_chunk_scan(x.float() * dt[..., None], A * dt, b.float(), c.float(), self.chunk_size)
        y = y + x.float() * self.D.float()[:, None]
        if cache is not None:
            k = self.conv_kernel_size
            window = F.pad(conv_in, (max(k - conv_in.shape[-1], 0), 0))[..., -k:]
            cache.update(conv_state=window, ssm_state=final_state, num_tokens_added=u.shape[1], layer_idx=self.layer_idx)
        y = y.reshape(*y.shape[:2], self.intermediate_size).to(dtype)
        return self.out_proj(self.norm(y, gate))

    def _step(self, u: torch.Tensor, cache) -> torch.Tensor:
        """u ``[B, 1, hidden]`` with an existing cache."""
        dtype = u.dtype
        conv_state, ssm_state = cache.get_cache(self.layer_idx)
        gate, xbc, dt = self._split(self.in_proj(u[:, 0]))
        conv_state = torch.cat([conv_state[..., 1:], xbc.unsqueeze(-1)], dim=-1)
        conv_out = (conv_state * self.conv1d.weight.squeeze(1)).sum(-1)
        if self.conv1d.bias is not None:
            conv_out = conv_out + self.conv1d.bias
        x, b, c, dt = self._ssm_inputs(self.activation(conv_out), dt)
        A = -torch.exp(self.A_log.float())
        decay = torch.exp(dt * A)  # [B, H]
        ssm_state = ssm_state * decay[..., None, None] + torch.einsum("bh,bhp,bhn->bhpn", dt, x.float(), b.float())
        y = torch.einsum("bhpn,bhn->bhp", ssm_state, c.float()) + x.float() * self.D.float()[:, None]
        cache.update(conv_state=conv_state, ssm_state=ssm_state, num_tokens_added=1, layer_idx=self.layer_idx)
        y = y.reshape(y.shape[0], 1, self.intermediate_size).to(dtype)
        return self.out_proj(self.norm(y, gate.unsqueeze(1)))

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        if ctx.packed and hidden_states.is_cuda and self._silu_activation and self.conv_kernel_size <= 8 and self._scan_kernel_ok(hidden_states):
            # all documents in one pass: the convolution and the scan kernels take the document boundaries from cu_seqlens
            return self._sequence(hidden_states.unsqueeze(0), None, None, cu_seqlens=ctx.cu_seqlens_int32()).squeeze(0)
        if ctx.packed:
            bounds = ctx.cu_seqlens.tolist()
            pieces = [self._sequence(hidden_states[s:e].unsqueeze(0), None, None).squeeze(0)
                      for s, e in zip(bounds[:-1], bounds[1:]) if e > s]
            return torch.cat(pieces, dim=0)
        if past_key_values is not None and past_key_values.get_seq_length(self.layer_idx) > 0 and hidden_states.shape[1] == 1:
            return self._step(hidden_states, past_key_values)
        mask = None
        if ctx.attention_mask is not None and not bool(torch.all(ctx.attention_mask == 1)):
            mask = ctx.attention_mask[:, -hidden_states.shape[1]:]
            hidden_states = hidden_states * mask[..., None].to(hidden_states.dtype)
        return self._sequence(hidden_states, mask, past_key_values)

"""Stick-breaking attention (arXiv 2410.17980): no positional embedding, no softmax.

For query i and key j < i (strictly causal): ``A_ij = sigmoid(z_ij) * prod_{j<k<i} (1 - sigmoid(z_ik))`` with
``z = scale * q k^T``; the mass that is left, ``rem_i = 1 - sum_j A_ij``, goes to a learned per-head vector
``head_bias``. The mixed heads are normalised with a GroupNorm (one group per head) before ``c_proj``.

Parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/stickbreaking_attention.py:20-224 (parameter names
``head_bias``, ``norm``). The math below is evaluated in fp32 as a dense ``[heads, q, k]`` problem per document: the
log of the running product is a reversed cumulative sum of ``logsigmoid(-z)`` over the keys between j and i.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..context import SequenceContext
from .attention import Attention


def stickbreaking_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """q ``[h, n_q, d]``, k / v ``[h, n_k, d]`` with the queries being the LAST ``n_q`` positions of the ``n_k`` keys.
    Returns ``(out [h, n_q, d], rem [h, n_q])``."""
    n_q, n_k = q.shape[1], k.shape[1]
    z = torch.einsum("hqd,hkd->hqk", q.float(), k.float()) * scale
    qi = torch.arange(n_k - n_q, n_k, device=q.device)[:, None]
    kj = torch.arange(n_k, device=q.device)[None, :]
    allowed = (kj < qi)[None]
    log_beta = F.logsigmoid(z)
    log_keep = F.logsigmoid(-z).masked_fill(~allowed, 0.0)
    # sum over k in (j, i): total over allowed keys minus the inclusive prefix up to j
    suffix = log_keep.sum(-1, keepdim=True) - log_keep.cumsum(-1)
    att = torch.exp(log_beta + suffix).masked_fill(~allowed, 0.0)
    rem = 1.0 - att.sum(-1)
    out = torch.einsum("hqk,hkd->hqd", att, v.float())
    return out.to(q.dtype), rem.to(q.dtype)


class _FusedStickBreaking(torch.autograd.Function):
    """The sm_100a kernels on the fused qkv buffer of a packed batch (``csrc/ops/sb_attention_{fwd,bwd}.cu``): forward
    walks the key tiles from the diagonal to the start of the document, backward does the same walk per query tile and
    reduces the key / value gradients across query tiles in fp32."""

    @staticmethod
    def forward(ctx, qkv, cu_seqlens, groups, group_size, head_dim, scale):
        from ... import ops

        out, rem = ops.native().sb_attn_fwd(qkv, cu_seqlens, groups, group_size, head_dim, scale, ops.status_word(qkv.device))
        ctx.save_for_backward(qkv, cu_seqlens, out, rem)
        ctx.meta = (groups, group_size, head_dim, scale)
        return out, rem

    @staticmethod
    def backward(ctx, d_out, d_rem):
        from ... import ops

        qkv, cu_seqlens, out, rem = ctx.saved_tensors
        groups, g, d, scale = ctx.meta
        if d_rem is None:
            d_rem = torch.zeros_like(rem)
        d_qkv = ops.native().sb_attn_bwd(d_out.contiguous(), d_rem.float().contiguous(), qkv, out, rem, cu_seqlens, groups, g, d, scale,
                                         ops.status_word(qkv.device))
        return d_qkv, None, None, None, None, None


class StickBreakingAttention(Attention):
    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int,
                 attention_multiplier: float | None, add_bias: bool, dropout: float, init_method: str,
                 initializer_range: float, m_width: float | None, num_layers: int, causal: bool, layer_idx: int | None,
                 use_padding_free_transformer: bool) -> None:
        super().__init__(hidden_size=hidden_size, num_attention_heads=num_attention_heads,
                         num_key_value_heads=num_key_value_heads, attention_multiplier=attention_multiplier,
                         position_embedding_type="nope", add_bias=add_bias, softmax_dropout=0, dropout=dropout,
                         init_method=init_method, initializer_range=initializer_range, m_width=m_width,
                         num_layers=num_layers, causal=causal, layer_idx=layer_idx,
                         use_padding_free_transformer=use_padding_free_transformer)
        self.head_bias = nn.Parameter(torch.zeros(self.num_heads, self.head_dim))
        self.norm = nn.GroupNorm(self.num_heads, self.hidden_size)

    def _kernel_ok(self, qkv: torch.Tensor) -> bool:
        from ... import ops
        from ...enums import Kernel
        from ...kernels import is_kernel_allowed

        from ...ops.attention import padded_head_dim

        return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and padded_head_dim(self.head_dim) is not None and ops.native_available()
                and hasattr(ops.native(), "sb_attn_fwd") and is_kernel_allowed(Kernel.stickbreaking_attention))

    def _heads(self, qkv: torch.Tensor):
        """``[n, C] -> q [hq, n, d], k / v [hq, n, d]`` (keys and values repeated over their query group)."""
        n = qkv.shape[0]
        g, hkv, d = self.group_size, self.num_key_value_heads, self.head_dim
        v4 = qkv.view(n, hkv, g + 2, d)
        q = v4[:, :, :g].reshape(n, hkv * g, d).transpose(0, 1)
        k = v4[:, :, g].repeat_interleave(g, dim=1).transpose(0, 1)
        v = v4[:, :, g + 1].repeat_interleave(g, dim=1).transpose(0, 1)
        return q, k, v

    def _mix(self, q, k, v) -> torch.Tensor:
        out, rem = stickbreaking_attention(q, k, v, self.softmax_scale)
        out = out + rem[..., None] * self.head_bias[:, None, :].to(out.dtype)
        return out.transpose(0, 1).reshape(q.shape[1], self.hidden_size)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        qkv = self.c_attn(hidden_states)
        if ctx.packed and self._kernel_ok(qkv):
            from ...ops.attention import pad_fused_qkv, padded_head_dim

            tokens = qkv.shape[0]
            width = padded_head_dim(self.head_dim)
            if width != self.head_dim:
                # head widths between the kernel widths (80, 96) run on the wider kernel over zero-padded heads
                qkv = pad_fused_qkv(qkv.contiguous(), self.num_key_value_heads, self.group_size, self.head_dim, width)
            out, rem = _FusedStickBreaking.apply(qkv.contiguous(), ctx.cu_seqlens_int32(), self.num_key_value_heads, self.group_size,
                                                 width, self.softmax_scale)
            out = out.view(tokens, self.num_heads, width)[:, :, : self.head_dim]
            mixed = out + rem.t().unsqueeze(-1).to(out.dtype) * self.head_bias.to(out.dtype)
            mixed = self.norm(mixed.reshape(tokens, self.hidden_size))
        elif ctx.packed:
            from ... import ops

            ops.note_fallback("stickbreaking_attention", f"head_dim {self.head_dim} or the kernel is not enabled", qkv)
            bounds = ctx.cu_seqlens.tolist()
            pieces = [self._mix(*self._heads(qkv[s:e])) for s, e in zip(bounds[:-1], bounds[1:]) if e > s]
            mixed = torch.cat(pieces, dim=0)
            mixed = self.norm(mixed)
        else:
            b, s, _ = qkv.shape
            parts = [self._heads(qkv[i]) for i in range(b)]
            q = torch.stack([p[0] for p in parts])
            k = torch.stack([p[1] for p in parts])
            v = torch.stack([p[2] for p in parts])
            if past_key_values is not None:
                k, v = past_key_values.update(key_states=k, value_states=v, layer_idx=self.layer_idx)
            mixed = torch.stack([self._mix(q[i], k[i], v[i]) for i in range(b)])
            mixed = self.norm(mixed.view(b * s, self.hidden_size)).view(b, s, self.hidden_size)
        return self.dropout(self.c_proj(mixed))

"""Causal softmax attention with a fused QKV projection (MHA / GQA / MQA).

Parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/softmax_attention.py:22-458. The rows of
``c_attn.weight`` are laid out per key/value group as ``[q heads of the group | k | v]`` - that is ``[q|k|v]`` per
head for MHA and ``[Q; k; v]`` for MQA - which is the checkpoint layout of the reference. ``c_proj`` is initialised
with ``std / sqrt(2 * num_layers)``.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...enums import Kernel
from ...kernels import is_kernel_allowed, wait_for_ACT
from ...ops.attention import attention_fused_qkv, split_fused_qkv
from ...utils import divide_if_divisible
from ..context import SequenceContext
from ..parameter import mark_parameter_as_mup_learning_rate
from .basic import ParameterizedLinear, dropout
from .rope import apply_rotary_pos_emb


# ----------------------------------------------------------------------------- layout helpers (HF import/export)
def interleave_query_key_value_tensor_for_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                                    num_heads: int, num_key_value_heads: int, head_dim: int) -> torch.Tensor:
    """Stack separate q/k/v projection weights (or biases) into the fused per-group layout."""
    g = divide_if_divisible(num_heads, num_key_value_heads, "")
    rest = q.shape[1:]
    qg = q.reshape(num_key_value_heads, g * head_dim, *rest)
    kg = k.reshape(num_key_value_heads, head_dim, *rest)
    vg = v.reshape(num_key_value_heads, head_dim, *rest)
    return torch.cat([qg, kg, vg], dim=1).reshape(-1, *rest)


def split_query_key_value_tensor_for_attention(qkv: torch.Tensor, num_heads: int, num_key_value_heads: int,
                                               head_dim: int | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Inverse of :func:`interleave_query_key_value_tensor_for_attention`."""
    g = divide_if_divisible(num_heads, num_key_value_heads, "")
    if head_dim is None:
        head_dim = qkv.shape[0] // (num_heads + 2 * num_key_value_heads)
    rest = qkv.shape[1:]
    grouped = qkv.reshape(num_key_value_heads, (g + 2) * head_dim, *rest)
    q, k, v = grouped.split((g * head_dim, head_dim, head_dim), dim=1)
    return q.reshape(-1, *rest), k.reshape(-1, *rest), v.reshape(-1, *rest)


def get_attention_head_type(num_attention_heads: int, num_key_value_heads: int) -> str:
    """"mha" (a key/value head per query head), "mqa" (one key/value head) or "gqa" (anything between); the names the
    tensor-parallel weight layout and the conversion tools go by."""
    return {1: "mqa", num_attention_heads: "mha"}.get(num_key_value_heads, "gqa")  # one head of each kind counts as "mha"


def repeat_key_value(x: torch.Tensor, num_heads: int, num_key_value_heads: int) -> torch.Tensor:
    """``[b, hkv, s, d] -> [b, hq, s, d]`` by repeating each key/value head for its query group."""
    g = num_heads // num_key_value_heads
    return x if g == 1 else x.repeat_interleave(g, dim=1)


class Attention(nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int,
                 attention_multiplier: float | None, position_embedding_type: str, add_bias: bool,
                 softmax_dropout: float, dropout: float, init_method: str, initializer_range: float,
                 m_width: float | None, num_layers: int, causal: bool, layer_idx: int | None,
                 use_padding_free_transformer: bool) -> None:
        super().__init__()
        self.causal = causal
        self.hidden_size = hidden_size
        self.num_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads
        self.add_bias = add_bias
        self.use_padding_free_transformer = use_padding_free_transformer
        self.head_dim = divide_if_divisible(hidden_size, num_attention_heads, "hidden_size must be divisible by num_attention_heads")
        self.group_size = divide_if_divisible(num_attention_heads, num_key_value_heads, "num_attention_heads must be divisible by num_key_value_heads")
        self.position_embedding_type = position_embedding_type
        self.attention_multiplier = attention_multiplier
        self.layer_idx = layer_idx

        std = initializer_range / math.sqrt(m_width) if init_method == "mup" else initializer_range
        self.c_attn = ParameterizedLinear(hidden_size, hidden_size + 2 * num_key_value_heads * self.head_dim, bias=add_bias, std=std)
        std = initializer_range / math.sqrt(2 * num_layers)
        if init_method == "mup":
            std /= math.sqrt(m_width)
        self.c_proj = ParameterizedLinear(hidden_size, hidden_size, bias=add_bias, std=std)

        self.softmax_dropout_p = softmax_dropout
        self.dropout = nn.Identity() if dropout == 0 else nn.Dropout(dropout)
        mark_parameter_as_mup_learning_rate(self.c_attn.weight)
        mark_parameter_as_mup_learning_rate(self.c_proj.weight)

    @property
    def softmax_scale(self) -> float:
        return self.attention_multiplier if self.attention_multiplier is not None else 1.0 / math.sqrt(self.head_dim)

    def _use_flash(self) -> bool:
        return is_kernel_allowed(Kernel.flash_attention_2) or is_kernel_allowed(Kernel.flash_attention_3)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        qkv = self.c_attn(hidden_states)
        if ctx.packed:
            out = self._forward_packed(qkv, ctx)
        else:
            out = self._forward_padded(qkv, ctx, past_key_values)
        out = self.c_proj(out)
        return self.dropout(out)

    # -------------------------------------------------------------- packed: [T, *]
    def _forward_packed(self, qkv: torch.Tensor, ctx: SequenceContext) -> torch.Tensor:
        g, hkv, d = self.group_size, self.num_key_value_heads, self.head_dim
        p_drop = self.softmax_dropout_p if self.training else 0.0
        if self.position_embedding_type == "rope":
            cos_h, sin_h = ctx.rope_half_tables
            qkv = ops.rope_fused_qkv(qkv, cos_h, sin_h, ctx.position_ids, hkv, g, d, cos_h.shape[-1] * 2)
        qkv = wait_for_ACT(qkv, wait_in_forward=True, wait_in_backward=False)
        out = attention_fused_qkv(qkv, ctx.cu_seqlens, ctx.max_seqlen, hkv, g, d, self.softmax_scale, self.causal, p_drop)
        return wait_for_ACT(out, wait_in_forward=False, wait_in_backward=True)

    # -------------------------------------------------------------- padded: [b, s, *]
    def _padded_on_varlen_kernels(self, qkv: torch.Tensor, ctx: SequenceContext) -> torch.Tensor | None:
        """A padded batch without a KV cache on the packed-sequence kernels: rotate the fused buffer in place of splitting
        it, drop the padding rows (``pack_sequence``), run the variable-length attention kernels, and put the rows back
        (the role of unpad -> flash_attn_varlen -> pad in lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/
        attention.py of the reference). Returns None when the batch does not qualify."""
        from ...ops.attention import _native_attention_ok
        from ...ops.sequence import compute_cu_seqlens_and_max_seqlen_from_attention_mask, pack_sequence, unpack_sequence

        b, s, width = qkv.shape
        g, hkv, d = self.group_size, self.num_key_value_heads, self.head_dim
        if not (self.causal and self._use_flash() and _native_attention_ok(qkv, d)):
            return None
        if self.training and self.softmax_dropout_p > 0:
            return None
        flat = qkv.reshape(b * s, width)
        if self.position_embedding_type == "rope":
            cos_h, sin_h = ctx.rope_half_tables
            position_ids = ctx.position_ids.expand(b, s).reshape(-1)
            flat = ops.rope_fused_qkv(flat, cos_h, sin_h, position_ids, hkv, g, d, cos_h.shape[-1] * 2)
        mask = ctx.attention_mask
        if mask is None:
            cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32, device=qkv.device)
            out = attention_fused_qkv(flat, cu, s, hkv, g, d, self.softmax_scale, True, 0.0)
            return out.view(b, s, hkv * g * d)
        cu, max_seqlen = compute_cu_seqlens_and_max_seqlen_from_attention_mask(mask)
        side = "left" if bool(mask[:, -1].all()) else "right"  # a batch is padded on one side as a whole
        packed = pack_sequence(flat.view(b, s, width), cu, side)
        out = attention_fused_qkv(packed, cu, max_seqlen, hkv, g, d, self.softmax_scale, True, 0.0)
        return unpack_sequence(out, cu, (b, s, hkv * g * d), side)

    def _forward_padded(self, qkv: torch.Tensor, ctx: SequenceContext, past_key_values) -> torch.Tensor:
        if past_key_values is None and qkv.is_cuda:
            out = self._padded_on_varlen_kernels(qkv, ctx)
            if out is not None:
                return out
        b, s, _ = qkv.shape
        g, hkv, d = self.group_size, self.num_key_value_heads, self.head_dim
        v5 = qkv.view(b, s, hkv, g + 2, d)
        q = v5[:, :, :, :g].reshape(b, s, hkv * g, d).transpose(1, 2)
        k = v5[:, :, :, g].transpose(1, 2)
        v = v5[:, :, :, g + 1].transpose(1, 2)
        if self.position_embedding_type == "rope":
            q = apply_rotary_pos_emb(q, ctx.rope_cos_sin)
            k = apply_rotary_pos_emb(k, ctx.rope_cos_sin)
        if past_key_values is not None:
            k, v = past_key_values.update(key_states=k, value_states=v, layer_idx=self.layer_idx)
        p_drop = self.softmax_dropout_p if self.training else 0.0
        mask = ctx.boolean_attention_mask(q.device)
        out = F.scaled_dot_product_attention(
            q, k, v, attn_mask=mask, dropout_p=p_drop, is_causal=self.causal and mask is None and q.shape[2] > 1,
            scale=self.softmax_scale, enable_gqa=g > 1,
        )
        return out.transpose(1, 2).reshape(b, s, hkv * g * d)

"""Multi-head latent attention: queries and keys/values pass through low-rank bottlenecks and the compressed
key/value stream is what the generation cache stores (parity:
lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/multihead_latent_attention.py:19-221; no-RoPE only)."""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.attention import attention_varlen_reference
from ..context import SequenceContext
from ..parameter import mark_parameter_as_mup_learning_rate
from .basic import ParameterizedLinear
from .normalization import get_normalization_function


class MultiHeadLatentAttention(nn.Module):
    def __init__(self, hidden_size: int, query_compression_size: int, key_value_compression_size: int,
                 num_attention_heads: int, head_dim: int, attention_multiplier: float | None,
                 position_embedding_type: str, add_bias: bool, softmax_dropout: float, dropout: float, init_method: str,
                 initializer_range: float, m_width: float | None, num_layers: int, causal: bool, layer_idx: int | None,
                 use_padding_free_transformer: bool, normalization_function: str = "layernorm",
                 layer_norm_epsilon: float = 1e-5) -> None:
        super().__init__()
        if position_embedding_type == "rope":
            raise NotImplementedError("multi-head latent attention is implemented for models without RoPE")
        self.causal = causal
        self.hidden_size = hidden_size
        self.num_heads = num_attention_heads
        self.head_dim = head_dim
        self.attention_multiplier = attention_multiplier
        self.layer_idx = layer_idx
        self.use_padding_free_transformer = use_padding_free_transformer
        std = initializer_range / (math.sqrt(m_width) if init_method == "mup" else 1)
        width = num_attention_heads * head_dim
        self.query_down_projection = ParameterizedLinear(hidden_size, query_compression_size, bias=add_bias, std=std)
        self.query_ln = get_normalization_function(normalization_function, query_compression_size, eps=layer_norm_epsilon)
        self.query_up_projection = ParameterizedLinear(query_compression_size, width, bias=add_bias, std=std)
        self.key_value_down_projection = ParameterizedLinear(hidden_size, 2 * key_value_compression_size, bias=add_bias, std=std)
        self.key_value_ln = get_normalization_function(normalization_function, 2 * key_value_compression_size, eps=layer_norm_epsilon)
        self.key_up_projection = ParameterizedLinear(key_value_compression_size, width, bias=add_bias, std=std)
        self.value_up_projection = ParameterizedLinear(key_value_compression_size, width, bias=add_bias, std=std)
        out_std = initializer_range / math.sqrt(2 * num_layers) / (math.sqrt(m_width) if init_method == "mup" else 1)
        self.c_proj = ParameterizedLinear(width, hidden_size, bias=add_bias, std=out_std)
        self.softmax_dropout_p = softmax_dropout
        self.softmax_dropout = nn.Identity() if softmax_dropout == 0 else nn.Dropout(softmax_dropout)
        self.dropout = nn.Identity() if dropout == 0 else nn.Dropout(dropout)
        for m in (self.query_down_projection, self.query_up_projection, self.key_value_down_projection,
                  self.key_up_projection, self.value_up_projection, self.c_proj):
            mark_parameter_as_mup_learning_rate(m.weight)

    @property
    def softmax_scale(self) -> float:
        return self.attention_multiplier if self.attention_multiplier is not None else 1.0 / math.sqrt(self.head_dim)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        q = self.query_up_projection(self.query_ln(self.query_down_projection(hidden_states)))
        kv = self.key_value_ln(self.key_value_down_projection(hidden_states))
        if past_key_values is not None:
            kv, _ = past_key_values.update(key_states=kv, value_states=None, layer_idx=self.layer_idx, sequence_length_dimension=1)
        k_c, v_c = kv.chunk(2, dim=-1)
        k = self.key_up_projection(k_c)
        v = self.value_up_projection(v_c)
        p_drop = self.softmax_dropout_p if self.training else 0.0
        if ctx.packed:
            T = q.shape[0]
            shape = (T, self.num_heads, self.head_dim)
            out = attention_varlen_reference(q.view(shape), k.view(shape), v.view(shape), ctx.cu_seqlens, self.softmax_scale,
                                             self.causal, p_drop).reshape(T, -1)
        else:
            b, s, _ = q.shape
            kl = k.shape[1]
            qh = q.view(b, s, self.num_heads, self.head_dim).transpose(1, 2)
            kh = k.view(b, kl, self.num_heads, self.head_dim).transpose(1, 2)
            vh = v.view(b, kl, self.num_heads, self.head_dim).transpose(1, 2)
            mask = ctx.boolean_attention_mask(q.device)
            out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, dropout_p=p_drop,
                                                 is_causal=self.causal and mask is None and s > 1, scale=self.softmax_scale)
            out = out.transpose(1, 2).reshape(b, s, -1)
        return self.dropout(self.c_proj(out))

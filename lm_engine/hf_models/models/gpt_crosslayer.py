"""``gpt_crosslayer``: cross-layer attention (arXiv 2405.12981). ``sharing_pattern[i] = j`` makes layer ``i`` attend
with the keys/values computed by layer ``j``; only layers with ``sharing_pattern[i] == i`` own a ``kv_proj`` (its own
norm ``kv_proj.ln`` + ``kv_proj.kv_attn`` with rows laid out per key/value head as ``[k | v]``). Every layer has a
query projection ``sequence_mixer.q_attn`` and ``sequence_mixer.c_proj``. RoPE is applied to the keys once where they
are produced and to the queries in every layer.

Parity: lm_engine/hf_models/models/gpt_crosslayer/{layer.py:23-125, base.py:13-75, sequence_mixers/base.py:23-238,
utils.py:14-141}.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.attention import attention_fused_qkv
from ...utils import divide_if_divisible
from ..cache import GenerationCache
from ..config import GPTBaseConfig, GPTCrossLayerConfig
from ..context import SequenceContext
from ..layers.attention import split_query_key_value_tensor_for_attention
from ..layers.basic import ParameterizedLinear
from ..layers.mixers import get_mlp_block
from ..layers.normalization import get_normalization_function
from ..layers.rope import apply_rotary_pos_emb
from ..modeling import BaseModelMixin, BaseModelOutputWithPast, CausalLMModelMixin, PreTrainedModelMixin
from ..utils import is_generation_cache_enabled


class KeyValueProjection(nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int, add_bias: bool,
                 initializer_range: float, normalization_function: str, layer_norm_epsilon: float) -> None:
        super().__init__()
        self.num_key_value_heads = num_key_value_heads
        self.head_dim = divide_if_divisible(hidden_size, num_attention_heads, "")
        self.ln = get_normalization_function(normalization_function, hidden_size, layer_norm_epsilon)
        self.kv_attn = ParameterizedLinear(hidden_size, 2 * num_key_value_heads * self.head_dim, bias=add_bias, std=initializer_range)

    def forward(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """-> k, v of shape ``[..., kv_heads, head_dim]`` (token dims leading)."""
        kv = self.kv_attn(self.ln(hidden_states))
        kv = kv.view(*kv.shape[:-1], self.num_key_value_heads, 2 * self.head_dim)
        return kv.split(self.head_dim, dim=-1)


class CrossLayerAttention(nn.Module):
    def __init__(self, config: GPTCrossLayerConfig, layer_idx: int, use_padding_free_transformer: bool) -> None:
        super().__init__()
        block = config.sequence_mixer_blocks[layer_idx]
        if block.sequence_mixer_type not in ("softmax_attention", "stickbreaking_attention"):
            raise ValueError("cross-layer attention is defined for softmax and stick-breaking attention layers")
        # stick-breaking layers (arXiv 2410.17980) share keys and values across layers the same way; they use no
        # positional embedding and carry the parameters of the stand-alone mixer (``head_bias``, ``norm``)
        self.stickbreaking = block.sequence_mixer_type == "stickbreaking_attention"
        self.hidden_size = config.hidden_size
        self.num_heads = block.num_attention_heads
        self.num_key_value_heads = block.num_key_value_heads
        self.head_dim = divide_if_divisible(self.hidden_size, self.num_heads, "")
        self.position_embedding_type = "nope" if self.stickbreaking else config.position_embedding_type
        self.attention_multiplier = block.attention_multiplier
        self.layer_idx = layer_idx
        self.softmax_dropout_p = getattr(block, "softmax_dropout", 0)
        if self.stickbreaking:
            self.head_bias = nn.Parameter(torch.zeros(self.num_heads, self.head_dim))
            self.norm = nn.GroupNorm(self.num_heads, self.hidden_size)
        std = config.initializer_range / (math.sqrt(config.m_width) if config.init_method == "mup" else 1)
        self.q_attn = ParameterizedLinear(self.hidden_size, self.hidden_size, bias=block.add_bias, std=std)
        self.c_proj = ParameterizedLinear(self.hidden_size, self.hidden_size, bias=block.add_bias,
                                          std=std / math.sqrt(2 * config.num_layers))
        self.dropout = nn.Identity() if block.dropout == 0 else nn.Dropout(block.dropout)

    @property
    def softmax_scale(self) -> float:
        return self.attention_multiplier if self.attention_multiplier is not None else 1.0 / math.sqrt(self.head_dim)

    # ------------------------------------------------------------------ stick-breaking
    def _stickbreaking_kernel_ok(self, q: torch.Tensor) -> bool:
        from ... import ops
        from ...enums import Kernel
        from ...kernels import is_kernel_allowed
        from ...ops.attention import padded_head_dim

        return (q.is_cuda and q.dtype == torch.bfloat16 and padded_head_dim(self.head_dim) is not None and ops.native_available()
                and hasattr(ops.native(), "sb_attn_fwd") and is_kernel_allowed(Kernel.stickbreaking_attention))

    def _stickbreaking_mix(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q ``[hq, n_q, d]``, k / v ``[hkv, n_k, d]`` of one document -> ``[n_q, hidden]`` (before the GroupNorm)."""
        from ..layers.stickbreaking import stickbreaking_attention

        group = self.num_heads // self.num_key_value_heads
        out, rem = stickbreaking_attention(q, k.repeat_interleave(group, dim=0), v.repeat_interleave(group, dim=0), self.softmax_scale)
        out = out + rem[..., None] * self.head_bias[:, None, :].to(out.dtype)
        return out.transpose(0, 1).reshape(q.shape[1], self.hidden_size)

    def _forward_stickbreaking(self, q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, ctx: SequenceContext) -> torch.Tensor:
        if ctx.packed:
            T = q.shape[0]
            q = q.view(T, self.num_heads, self.head_dim)
            if self._stickbreaking_kernel_ok(q):
                from ...ops.attention import pad_fused_qkv, padded_head_dim
                from ..layers.stickbreaking import _FusedStickBreaking

                groups, qpg = self.num_key_value_heads, self.num_heads // self.num_key_value_heads
                fused = torch.cat([q.view(T, groups, qpg, self.head_dim), key.reshape(T, groups, 1, self.head_dim).to(q.dtype),
                                   value.reshape(T, groups, 1, self.head_dim).to(q.dtype)], dim=2).reshape(T, groups * (qpg + 2) * self.head_dim)
                width = padded_head_dim(self.head_dim)
                if width != self.head_dim:
                    fused = pad_fused_qkv(fused, groups, qpg, self.head_dim, width)
                out, rem = _FusedStickBreaking.apply(fused.contiguous(), ctx.cu_seqlens_int32(), groups, qpg, width, self.softmax_scale)
                out = out.view(T, self.num_heads, width)[:, :, : self.head_dim]
                mixed = out + rem.t().unsqueeze(-1).to(out.dtype) * self.head_bias.to(out.dtype)
                mixed = mixed.reshape(T, self.hidden_size)
            else:
                bounds = ctx.cu_seqlens.tolist()
                mixed = torch.cat([self._stickbreaking_mix(q[s:e].transpose(0, 1), key[s:e].transpose(0, 1), value[s:e].transpose(0, 1))
                                   for s, e in zip(bounds[:-1], bounds[1:]) if e > s], dim=0)
            return self.norm(mixed)
        b, s, _ = q.shape
        q = q.view(b, s, self.num_heads, self.head_dim).transpose(1, 2)  # key / value arrive as [b, hkv, n_k, d]
        mixed = torch.stack([self._stickbreaking_mix(q[i], key[i], value[i]) for i in range(b)])
        return self.norm(mixed.view(b * s, self.hidden_size)).view(b, s, self.hidden_size)

    def forward(self, hidden_states: torch.Tensor, key: torch.Tensor, value: torch.Tensor, ctx: SequenceContext) -> torch.Tensor:
        q = self.q_attn(hidden_states)
        if self.stickbreaking:
            return self.dropout(self.c_proj(self._forward_stickbreaking(q, key, value, ctx)))
        p_drop = self.softmax_dropout_p if self.training else 0.0
        if ctx.packed:
            T = q.shape[0]
            q = q.view(T, self.num_heads, self.head_dim)
            if self.position_embedding_type == "rope":
                cos, sin = ctx.rope_cos_sin
                q = apply_rotary_pos_emb(q, (cos, sin))
            # One buffer laid out like a fused projection (per key/value group: its query heads, then k, then v), so that
            # the packed-sequence attention kernels serve this model too; the keys and values may come from another
            # layer (reference: lm_engine/hf_models/models/gpt_crosslayer/sequence_mixers in the reference calls flash
            # attention on the separate tensors).
            groups, qpg = self.num_key_value_heads, self.num_heads // self.num_key_value_heads
            fused = torch.cat([q.view(T, groups, qpg, self.head_dim), key.reshape(T, groups, 1, self.head_dim).to(q.dtype),
                               value.reshape(T, groups, 1, self.head_dim).to(q.dtype)], dim=2).reshape(T, groups * (qpg + 2) * self.head_dim)
            out = attention_fused_qkv(fused, ctx.cu_seqlens, ctx.max_seqlen, groups, qpg, self.head_dim, self.softmax_scale, True, p_drop)
        else:
            b, s, _ = q.shape
            q = q.view(b, s, self.num_heads, self.head_dim).transpose(1, 2)
            if self.position_embedding_type == "rope":
                q = apply_rotary_pos_emb(q, ctx.rope_cos_sin)
            mask = ctx.boolean_attention_mask(q.device)
            out = F.scaled_dot_product_attention(q, key, value, attn_mask=mask, dropout_p=p_drop,
                                                 is_causal=mask is None and s > 1, scale=self.softmax_scale,
                                                 enable_gqa=self.num_heads != self.num_key_value_heads)
            out = out.transpose(1, 2).reshape(b, s, -1)
        return self.dropout(self.c_proj(out))


class GPTCrossLayerBlock(nn.Module):
    def __init__(self, config: GPTCrossLayerConfig, use_padding_free_transformer: bool, layer_idx: int) -> None:
        super().__init__()
        self.m_residual = config.m_residual
        self.layer_idx = layer_idx
        block = config.sequence_mixer_blocks[layer_idx]
        self.position_embedding_type = "nope" if block.sequence_mixer_type == "stickbreaking_attention" else config.position_embedding_type
        self.kv_proj = None
        if config.sharing_pattern[layer_idx] == layer_idx:
            self.kv_proj = KeyValueProjection(config.hidden_size, block.num_attention_heads, block.num_key_value_heads,
                                              block.add_bias, config.initializer_range, config.normalization_function,
                                              config.layer_norm_epsilon)
        self.ln_1 = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.sequence_mixer = CrossLayerAttention(config, layer_idx, use_padding_free_transformer)
        self.ln_2 = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp_block = get_mlp_block(config, use_padding_free_transformer=use_padding_free_transformer, layer_idx=layer_idx)

    def forward(self, hidden_states, key, value, ctx: SequenceContext, past_key_values=None):
        if self.kv_proj is not None:
            key, value = self.kv_proj(hidden_states)
            if ctx.packed:
                if self.position_embedding_type == "rope":
                    key = apply_rotary_pos_emb(key, ctx.rope_cos_sin)
            else:
                key, value = key.transpose(1, 2), value.transpose(1, 2)
                if self.position_embedding_type == "rope":
                    key = apply_rotary_pos_emb(key, ctx.rope_cos_sin)
                if past_key_values is not None:
                    key, value = past_key_values.update(key_states=key, value_states=value, layer_idx=self.layer_idx)
        update = self.sequence_mixer(self.ln_1(hidden_states), key, value, ctx)
        if self.m_residual is not None:
            update = update * self.m_residual
        hidden_states = hidden_states + update
        update = self.mlp_block(self.ln_2(hidden_states))
        if self.m_residual is not None:
            update = update * self.m_residual
        return hidden_states + update, key, value


class GPTCrossLayerPreTrainedModel(PreTrainedModelMixin):
    config_class = GPTCrossLayerConfig
    layer_class = GPTCrossLayerBlock
    _no_split_modules = ["GPTCrossLayerBlock"]


class GPTCrossLayerModel(GPTCrossLayerPreTrainedModel, BaseModelMixin):
    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None, position_ids=None,
                inputs_embeds=None, use_cache=None, cu_seqlens=None, max_seqlen=None) -> BaseModelOutputWithPast:
        if use_cache is None:
            use_cache = False if self.use_padding_free_transformer else self.config.use_cache
        dtype = self.wte.weight.dtype
        ctx = self.build_context(input_ids, inputs_embeds, attention_mask, position_ids, past_key_values, cu_seqlens, max_seqlen, dtype)
        if ctx.packed and self.position_embedding_type == "rope":
            cos, sin = self.rope(max(ctx.max_seqlen, self.config.max_position_embeddings), dtype=dtype, device=ctx.cu_seqlens.device)
            ctx.rope_cos_sin = (cos[ctx.position_ids.long()].unsqueeze(1), sin[ctx.position_ids.long()].unsqueeze(1))
        hidden_states = self.embed(input_ids, inputs_embeds, ctx.position_ids, token_type_ids)
        if is_generation_cache_enabled() and use_cache and past_key_values is None:
            past_key_values = GenerationCache(self.config)
        key = value = None
        for block in self.h:
            hidden_states, key, value = block(hidden_states, key, value, ctx, past_key_values)
        return BaseModelOutputWithPast(last_hidden_state=self.ln_f(hidden_states), past_key_values=past_key_values)


class GPTCrossLayerForCausalLM(GPTCrossLayerPreTrainedModel, CausalLMModelMixin):
    base_model_class = GPTCrossLayerModel


def convert_gpt_base_to_gpt_crosslayer(original_config: GPTBaseConfig, original_model, sharing_pattern: list[int] | None = None,
                                       **kwargs):
    """Re-express a ``gpt_base`` model as ``gpt_crosslayer``. With the identity sharing pattern the converted model
    computes the same function; with sharing, layers that give up their keys/values simply lose those weights."""
    config = GPTCrossLayerConfig(
        vocab_size=original_config.vocab_size, max_position_embeddings=original_config.max_position_embeddings,
        hidden_size=original_config.hidden_size, num_layers=original_config.num_layers,
        embedding_dropout=original_config.embedding_dropout, normalization_function=original_config.normalization_function,
        layer_norm_epsilon=original_config.layer_norm_epsilon, position_embedding_type=original_config.position_embedding_type,
        rope_theta=original_config.rope_theta, use_cache=original_config.use_cache, sharing_pattern=sharing_pattern,
        tie_word_embeddings=original_config.tie_word_embeddings, initializer_range=original_config.initializer_range,
        m_emb=original_config.m_emb, m_width=original_config.m_width, m_residual=original_config.m_residual,
        bos_token_id=original_config.bos_token_id, eos_token_id=original_config.eos_token_id, pad_token_id=original_config.pad_token_id,
        sequence_mixer_blocks=[b.to_dict() for b in original_config.sequence_mixer_blocks],
        mlp_blocks=[b.to_dict() for b in original_config.mlp_blocks])
    model = GPTCrossLayerForCausalLM(config, **kwargs).to(next(original_model.parameters()).dtype)
    source = original_model.state_dict()
    target = {}
    heads = config.check_equal_for_all_and_get_value("sequence_mixer_blocks", "num_attention_heads")
    head_dim = config.hidden_size // heads
    for name, tensor in source.items():
        if ".sequence_mixer.c_attn." not in name and ".ln_1." not in name:
            target[name] = tensor
    for i in range(config.num_layers):
        kv_heads = config.sequence_mixer_blocks[i].num_key_value_heads
        prefix = f"transformer.h.{i}."
        for suffix in ("weight", "bias"):
            key = f"{prefix}sequence_mixer.c_attn.{suffix}"
            if key not in source:
                continue
            q, k, v = split_query_key_value_tensor_for_attention(source[key], heads, kv_heads, head_dim)
            target[f"{prefix}sequence_mixer.q_attn.{suffix}"] = q
            if config.sharing_pattern[i] == i:
                rest = k.shape[1:]
                kv = torch.cat([k.reshape(kv_heads, head_dim, *rest), v.reshape(kv_heads, head_dim, *rest)], dim=1)
                target[f"{prefix}kv_proj.kv_attn.{suffix}"] = kv.reshape(-1, *rest)
        for suffix in ("weight", "bias"):
            key = f"{prefix}ln_1.{suffix}"
            if key in source:
                target[key] = source[key]
                if config.sharing_pattern[i] == i:
                    target[f"{prefix}kv_proj.ln.{suffix}"] = source[key]
    model.load_state_dict(target)
    return config, model

"""``desync_residual``: single-process simulation of tensor parallel training in which some all-reduces are skipped.

Activations carry a leading dimension of size ``pretraining_tensor_parallel_size`` (one residual stream per simulated
rank). Attention heads and MLP columns are split over that dimension exactly as column/row parallel layers would
split them (:class:`DesyncResidualLinear` applies one weight slice per simulated rank with a batched product).
``reduce_pattern[layer] = {"attention": bool, "mlp": bool}`` says whether the partial outputs of a sub-block are
summed over the simulated ranks (a real all-reduce: every stream receives the full update) or whether every stream
only adds its own partial output and the streams drift apart. The streams are averaged before the final norm; with
an all-true pattern the model computes the same function as ``gpt_base`` with concatenated weights.

Parity: lm_engine/hf_models/models/desync_residual/* (research model; no real communication).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...utils import divide_if_divisible
from ..config import DesyncResidualConfig
from ..context import SequenceContext
from ..layers.basic import init_zeros_
from ..layers.activations import get_activation_function, is_glu
from ..layers.normalization import get_normalization_function
from ..layers.rope import apply_rotary_pos_emb
from ..modeling import BaseModelMixin, BaseModelOutputWithPast, CausalLMModelMixin, PreTrainedModelMixin
from ..parameter import mark_parameter_as_no_weight_decay


class DesyncResidualLinear(nn.Module):
    """``tp`` independent linear maps applied to ``tp`` inputs: weight ``[tp, out, in]``, input ``[tp, ..., in]``."""

    def __init__(self, in_features: int, out_features: int, tensor_parallel_size: int, bias: bool = True, std: float = 0.02) -> None:
        super().__init__()
        self.tp = tensor_parallel_size
        self.std = std
        self.weight = nn.Parameter(torch.empty(tensor_parallel_size, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(tensor_parallel_size, out_features)) if bias else None
        mark_parameter_as_no_weight_decay(self.bias)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0.0, std=self.std)
        init_zeros_(self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[1:-1]
        y = torch.bmm(x.reshape(self.tp, -1, x.shape[-1]), self.weight.transpose(1, 2))
        if self.bias is not None:
            y = y + self.bias[:, None, :]
        return y.reshape(self.tp, *lead, -1)


def _combine(partial: torch.Tensor, reduce: bool) -> torch.Tensor:
    """A real all-reduce gives every simulated rank the sum; without it each rank keeps its own partial output."""
    return partial.sum(dim=0, keepdim=True).expand_as(partial) if reduce else partial


class DesyncResidualAttention(nn.Module):
    def __init__(self, config: DesyncResidualConfig, layer_idx: int) -> None:
        super().__init__()
        block = config.sequence_mixer_blocks[layer_idx]
        self.tp = config.pretraining_tensor_parallel_size
        self.layer_idx = layer_idx
        self.num_heads = block.num_attention_heads
        self.num_key_value_heads = block.num_key_value_heads
        self.head_dim = divide_if_divisible(config.hidden_size, self.num_heads, "")
        self.heads_per_rank = divide_if_divisible(self.num_heads, self.tp, "heads must divide over the simulated ranks")
        self.kv_per_rank = divide_if_divisible(self.num_key_value_heads, self.tp, "kv heads must divide over the simulated ranks")
        self.position_embedding_type = config.position_embedding_type
        self.attention_multiplier = block.attention_multiplier
        self.reduce = config.reduce_pattern[layer_idx]["attention"]
        width = (self.heads_per_rank + 2 * self.kv_per_rank) * self.head_dim
        self.c_attn = DesyncResidualLinear(config.hidden_size, width, self.tp, bias=block.add_bias, std=config.initializer_range)
        self.c_proj = DesyncResidualLinear(self.heads_per_rank * self.head_dim, config.hidden_size, self.tp, bias=block.add_bias,
                                           std=config.initializer_range / math.sqrt(2 * config.num_layers))

    def forward(self, x: torch.Tensor, ctx: SequenceContext) -> torch.Tensor:
        """x ``[tp, b, s, H]`` (padded batches only)."""
        tp, b, s, _ = x.shape
        g = self.heads_per_rank // self.kv_per_rank
        qkv = self.c_attn(x).view(tp * b, s, self.kv_per_rank, g + 2, self.head_dim)
        q = qkv[..., :g, :].reshape(tp * b, s, self.heads_per_rank, self.head_dim).transpose(1, 2)
        k = qkv[..., g, :].transpose(1, 2)
        v = qkv[..., g + 1, :].transpose(1, 2)
        if self.position_embedding_type == "rope":
            cos, sin = ctx.rope_cos_sin
            cos, sin = cos.repeat(tp, 1, 1, 1) if cos.shape[0] == b else cos, sin.repeat(tp, 1, 1, 1) if sin.shape[0] == b else sin
            q, k = apply_rotary_pos_emb(q, (cos, sin)), apply_rotary_pos_emb(k, (cos, sin))
        mask = ctx.boolean_attention_mask(x.device)
        if mask is not None:
            mask = mask.repeat(tp, 1, 1, 1)
        scale = self.attention_multiplier if self.attention_multiplier is not None else 1.0 / math.sqrt(self.head_dim)
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=mask is None and s > 1, scale=scale, enable_gqa=g > 1)
        out = out.transpose(1, 2).reshape(tp, b, s, self.heads_per_rank * self.head_dim)
        return _combine(self.c_proj(out), self.reduce)


class DesyncResidualMLP(nn.Module):
    def __init__(self, config: DesyncResidualConfig, layer_idx: int) -> None:
        super().__init__()
        block = config.mlp_blocks[layer_idx]
        self.tp = config.pretraining_tensor_parallel_size
        self.reduce = config.reduce_pattern[layer_idx]["mlp"]
        inter = divide_if_divisible(block.intermediate_size, self.tp, "intermediate size must divide over the simulated ranks")
        gated = is_glu(block.activation_function)
        self.c_fc = DesyncResidualLinear(config.hidden_size, (2 if gated else 1) * inter, self.tp, bias=block.add_bias, std=config.initializer_range)
        self.act = get_activation_function(block.activation_function)
        self.c_proj = DesyncResidualLinear(inter, config.hidden_size, self.tp, bias=block.add_bias,
                                           std=config.initializer_range / math.sqrt(2 * config.num_layers))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _combine(self.c_proj(self.act(self.c_fc(x))), self.reduce)


class DesyncResidualBlock(nn.Module):
    def __init__(self, config: DesyncResidualConfig, use_padding_free_transformer: bool, layer_idx: int) -> None:
        super().__init__()
        if use_padding_free_transformer:
            raise NotImplementedError("desync_residual runs on padded batches")
        self.m_residual = config.m_residual
        self.ln_1 = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.sequence_mixer = DesyncResidualAttention(config, layer_idx)
        self.ln_2 = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp_block = DesyncResidualMLP(config, layer_idx)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        update = self.sequence_mixer(self.ln_1(hidden_states), ctx)
        hidden_states = hidden_states + (update if self.m_residual is None else update * self.m_residual)
        update = self.mlp_block(self.ln_2(hidden_states))
        return hidden_states + (update if self.m_residual is None else update * self.m_residual)


class DesyncResidualPreTrainedModel(PreTrainedModelMixin):
    config_class = DesyncResidualConfig
    layer_class = DesyncResidualBlock
    _no_split_modules = ["DesyncResidualBlock"]


class DesyncResidualModel(DesyncResidualPreTrainedModel, BaseModelMixin):
    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None, position_ids=None,
                inputs_embeds=None, use_cache=None, cu_seqlens=None, max_seqlen=None) -> BaseModelOutputWithPast:
        if past_key_values is not None or use_cache:
            raise NotImplementedError("desync_residual is a training-time research model without a generation cache")
        ctx = self.build_context(input_ids, inputs_embeds, attention_mask, position_ids, None, cu_seqlens, max_seqlen, self.wte.weight.dtype)
        hidden_states = self.embed(input_ids, inputs_embeds, ctx.position_ids, token_type_ids)
        tp = self.config.pretraining_tensor_parallel_size
        hidden_states = hidden_states.unsqueeze(0).expand(tp, *hidden_states.shape)
        for block in self.h:
            hidden_states = block(hidden_states, ctx)
        return BaseModelOutputWithPast(last_hidden_state=self.ln_f(hidden_states.mean(dim=0)), past_key_values=None)


class DesyncResidualForCausalLM(DesyncResidualPreTrainedModel, CausalLMModelMixin):
    base_model_class = DesyncResidualModel

    def forward(self, *args, use_cache=None, **kwargs):
        return super().forward(*args, use_cache=False, **kwargs)

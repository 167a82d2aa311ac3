"""``ladder_residual``: every block works on a residual stream that is one update behind - the attention and MLP
outputs of block ``i`` are only added to the stream inside block ``i + 1``. Under tensor parallelism this lets the
all-reduce of an output overlap with the next sub-block's compute
(parity: lm_engine/hf_models/models/ladder_residual/{layer.py:11-48, base.py:13-94})."""

from __future__ import annotations

import torch

from ..cache import GenerationCache
from ..config import LadderResidualConfig
from ..context import SequenceContext
from ..modeling import BaseModelMixin, BaseModelOutputWithPast, Block, CausalLMModelMixin, PreTrainedModelMixin
from ..utils import is_generation_cache_enabled


class LadderResidualBlock(Block):
    def forward(self, current_attention_out, current_mlp_out, residual: torch.Tensor, ctx: SequenceContext,
                past_key_values=None):
        if current_attention_out is not None:
            residual = residual + current_attention_out
        current_attention_out = self.sequence_mixer(self.ln_1(residual), ctx, past_key_values)
        if self.m_residual is not None:
            current_attention_out = current_attention_out * self.m_residual
        if current_mlp_out is not None:
            residual = residual + current_mlp_out
        current_mlp_out = self.mlp_block(self.ln_2(residual))
        if self.m_residual is not None:
            current_mlp_out = current_mlp_out * self.m_residual
        return current_attention_out, current_mlp_out, residual


class LadderResidualPreTrainedModel(PreTrainedModelMixin):
    config_class = LadderResidualConfig
    layer_class = LadderResidualBlock
    _no_split_modules = ["LadderResidualBlock"]


class LadderResidualModel(LadderResidualPreTrainedModel, BaseModelMixin):
    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None, position_ids=None,
                inputs_embeds=None, use_cache=None, cu_seqlens=None, max_seqlen=None) -> BaseModelOutputWithPast:
        if use_cache is None:
            use_cache = False if self.use_padding_free_transformer else self.config.use_cache
        ctx = self.build_context(input_ids, inputs_embeds, attention_mask, position_ids, past_key_values, cu_seqlens,
                                 max_seqlen, self.wte.weight.dtype)
        residual = self.embed(input_ids, inputs_embeds, ctx.position_ids, token_type_ids)
        if is_generation_cache_enabled() and use_cache and past_key_values is None:
            past_key_values = GenerationCache(self.config)
        attention_out = mlp_out = None
        for block in self.h:
            attention_out, mlp_out, residual = block(attention_out, mlp_out, residual, ctx, past_key_values)
        hidden_states = self.ln_f(residual + attention_out + mlp_out)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=past_key_values)


class LadderResidualForCausalLM(LadderResidualPreTrainedModel, CausalLMModelMixin):
    base_model_class = LadderResidualModel

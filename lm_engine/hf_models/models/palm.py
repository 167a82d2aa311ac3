"""``palm``: parallel block - attention and MLP read the same normalised input and their sum joins the residual
stream (parity: lm_engine/hf_models/models/palm/{layer.py:13-60, base.py, main.py})."""

from __future__ import annotations

import torch
import torch.nn as nn

from ..config import PaLMConfig
from ..context import SequenceContext
from ..layers.mixers import get_mlp_block, get_sequence_mixer
from ..layers.normalization import get_normalization_function
from ..modeling import BaseModelMixin, CausalLMModelMixin, PreTrainedModelMixin


class PaLMBlock(nn.Module):
    def __init__(self, config: PaLMConfig, use_padding_free_transformer: bool, layer_idx: int | None = None) -> None:
        super().__init__()
        self.m_residual = config.m_residual
        self.ln = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.sequence_mixer = get_sequence_mixer(config, True, use_padding_free_transformer, layer_idx)
        self.mlp_block = get_mlp_block(config, use_padding_free_transformer=use_padding_free_transformer, layer_idx=layer_idx)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values=None) -> torch.Tensor:
        normed = self.ln(hidden_states)
        update = self.sequence_mixer(normed, ctx, past_key_values) + self.mlp_block(normed)
        if self.m_residual is not None:
            update = update * self.m_residual
        return hidden_states + update


class PaLMPreTrainedModel(PreTrainedModelMixin):
    config_class = PaLMConfig
    layer_class = PaLMBlock
    _no_split_modules = ["PaLMBlock"]


class PaLMModel(PaLMPreTrainedModel, BaseModelMixin):
    ...


class PaLMForCausalLM(PaLMPreTrainedModel, CausalLMModelMixin):
    base_model_class = PaLMModel

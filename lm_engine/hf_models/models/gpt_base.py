"""``gpt_base``: the plain decoder (parity: lm_engine/hf_models/models/gpt_base/{base,main}.py)."""

from __future__ import annotations

from ..config import GPTBaseConfig
from ..modeling import BaseModelMixin, CausalLMModelMixin, PreTrainedModelMixin


class GPTBasePreTrainedModel(PreTrainedModelMixin):
    config_class = GPTBaseConfig


class GPTBaseModel(GPTBasePreTrainedModel, BaseModelMixin):
    ...


class GPTBaseForCausalLM(GPTBasePreTrainedModel, CausalLMModelMixin):
    base_model_class = GPTBaseModel

"""Registration of the custom model types with the transformers Auto* factories
(parity: lm_engine/hf_models/register_hf.py:29-66)."""

from __future__ import annotations

from transformers import AutoConfig, AutoModel, AutoModelForCausalLM

from .config import CommonConfig, DesyncResidualConfig, GPTBaseConfig, GPTCrossLayerConfig, LadderResidualConfig, PaLMConfig

_CUSTOM_MODEL_REGISTRY: list[tuple] = []
_CUSTOM_MODEL_TYPES: list[str] = []
_CUSTOM_MODEL_CLASSES: list[type] = []
_MODEL_PARALLEL_CLASS_MAPPING: dict[str, type] = {}


def _register(config_class, base_class, causal_class) -> None:
    model_type = config_class.model_type
    if model_type in _CUSTOM_MODEL_TYPES:
        return
    AutoConfig.register(model_type, config_class, exist_ok=True)
    AutoModel.register(config_class, base_class, exist_ok=True)
    AutoModelForCausalLM.register(config_class, causal_class, exist_ok=True)
    _CUSTOM_MODEL_TYPES.append(model_type)
    _CUSTOM_MODEL_CLASSES.append(causal_class)


def register_model_classes() -> None:
    from .models.gpt_base import GPTBaseForCausalLM, GPTBaseModel

    _register(GPTBaseConfig, GPTBaseModel, GPTBaseForCausalLM)
    try:
        from .models.gpt_crosslayer import GPTCrossLayerForCausalLM, GPTCrossLayerModel
        from .models.palm import PaLMForCausalLM, PaLMModel
        from .models.ladder_residual import LadderResidualForCausalLM, LadderResidualModel
        from .models.desync_residual import DesyncResidualForCausalLM, DesyncResidualModel

        _register(GPTCrossLayerConfig, GPTCrossLayerModel, GPTCrossLayerForCausalLM)
        _register(PaLMConfig, PaLMModel, PaLMForCausalLM)
        _register(LadderResidualConfig, LadderResidualModel, LadderResidualForCausalLM)
        _register(DesyncResidualConfig, DesyncResidualModel, DesyncResidualForCausalLM)
    except ImportError:
        pass
    try:
        from .models.tensor_parallel import GPTBaseForCausalLM_TP, LadderResidualForCausalLM_TP

        _MODEL_PARALLEL_CLASS_MAPPING["gpt_base"] = GPTBaseForCausalLM_TP
        _MODEL_PARALLEL_CLASS_MAPPING["ladder_residual"] = LadderResidualForCausalLM_TP
    except ImportError:
        pass


def is_custom_model(model_type: str) -> bool:
    return model_type in _CUSTOM_MODEL_TYPES


def get_model_parallel_class(model_type: str):
    if model_type in _MODEL_PARALLEL_CLASS_MAPPING:
        return _MODEL_PARALLEL_CLASS_MAPPING[model_type]
    raise ValueError(f"model parallelism is not supported with `model_type` ({model_type})")

"""Model family of this engine, registered with the transformers Auto* factories on import
(parity: lm_engine/hf_models/__init__.py:5-42)."""

from .cache import GenerationCache
from .config import (
    CommonConfig,
    DesyncResidualConfig,
    GPTBaseConfig,
    GPTCrossLayerConfig,
    LadderResidualConfig,
    PaLMConfig,
)
from .loss import (
    add_aux_loss,
    clear_aux_loss,
    get_autoregressive_language_modeling_loss,
    get_aux_loss,
    is_aux_loss_zero,
)
from .modeling import (
    BaseModelOutputWithPast,
    CausalLMOutputWithPast,
    PipelineParallelInput,
    PipelineParallelOutput,
)
from .models.gpt_base import GPTBaseForCausalLM, GPTBaseModel
from .parameter import (
    is_parameter_with_mup_learning_rate,
    is_parameter_with_no_weight_decay,
    mark_parameter_as_mup_learning_rate,
    mark_parameter_as_no_weight_decay,
)
from .register_hf import get_model_parallel_class, is_custom_model, register_model_classes
from .utils import convert_padding_free_lists_to_tensors, disable_generation_cache

register_model_classes()


def __getattr__(name: str):
    """Lazily resolved exports (models and tools that are only needed by some entry points)."""
    import importlib

    lazy = {
        "GPTCrossLayerForCausalLM": ".models.gpt_crosslayer", "GPTCrossLayerModel": ".models.gpt_crosslayer",
        "convert_gpt_base_to_gpt_crosslayer": ".models.gpt_crosslayer",
        "PaLMForCausalLM": ".models.palm", "PaLMModel": ".models.palm",
        "LadderResidualForCausalLM": ".models.ladder_residual", "LadderResidualModel": ".models.ladder_residual",
        "DesyncResidualForCausalLM": ".models.desync_residual", "DesyncResidualModel": ".models.desync_residual",
        "GPTBaseForCausalLM_TP": ".models.tensor_parallel", "GPTBaseModel_TP": ".models.tensor_parallel",
        "LadderResidualForCausalLM_TP": ".models.tensor_parallel", "LadderResidualModel_TP": ".models.tensor_parallel",
        "import_from_huggingface": ".model_conversion", "export_to_huggingface": ".model_conversion",
        "fix_unsharded_state_dict": ".tp_weights", "unshard_tensor_parallel_state_dicts": ".tp_weights",
    }
    if name in lazy:
        return getattr(importlib.import_module(lazy[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

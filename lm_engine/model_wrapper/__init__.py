"""Wrapper factory (parity: lm_engine/model_wrapper/__init__.py:24-72): one wrapper per local pipeline stage."""

from __future__ import annotations

from ..containers import ModelContainer
from ..enums import Mode, TuningMethod
from ..kernels import enable_kernels
from ..utils import get_pipeline_stage_ids_on_current_rank, string_to_torch_dtype
from .base import ModelWrapper
from .pretraining import ModelWrapperForPretraining

_WRAPPER_OF_TUNING_METHOD = {
    TuningMethod.pretraining: "pretraining",
    TuningMethod.full_finetuning: "finetuning",
    TuningMethod.distillation: "distillation",
}


def _wrapper_class(tuning_method: TuningMethod):
    if tuning_method == TuningMethod.pretraining:
        return ModelWrapperForPretraining
    if tuning_method == TuningMethod.full_finetuning:
        from .finetuning import ModelWrapperForFinetuning

        return ModelWrapperForFinetuning
    if tuning_method == TuningMethod.distillation:
        from .distillation import ModelWrapperForDistillation

        return ModelWrapperForDistillation
    raise ValueError(f"unexpected tuning_method ({tuning_method})")


def get_model_container(args, mode: Mode) -> ModelContainer:
    tuning_method = args.tuning_args.tuning_method
    num_stages = args.distributed_args.num_pipeline_stages
    if tuning_method != TuningMethod.pretraining and num_stages != 1:
        raise ValueError("pipeline parallel is only supported for pretraining")

    kwargs = dict(
        mode=mode,
        model_name=args.model_args.model_name,
        pretrained_config=args.model_args.pretrained_config,
        model_class=args.model_args.model_class,
        dtype=string_to_torch_dtype(args.mixed_precision_args.dtype),
        efficient_initialization=args.model_args.efficient_initialization,
        use_padding_free_transformer=args.model_args.use_padding_free_transformer,
        sequence_parallel=args.distributed_args.sequence_parallel,
        num_pipeline_stages=num_stages,
        trust_remote_code=args.model_args.trust_remote_code,
        tokenizer_name=args.tokenizer_args.tokenizer_name,
        additional_special_tokens=args.tokenizer_args.additional_special_tokens,
    )
    if tuning_method in (TuningMethod.pretraining, TuningMethod.distillation):
        kwargs["micro_batch_size"] = args.training_parameters.micro_batch_size
        kwargs["sequence_length"] = args.datasets[0].class_args.get("sequence_length")
        kwargs["reset_attention_mask"] = args.model_args.reset_attention_mask
        kwargs["reset_position_ids"] = args.model_args.reset_position_ids
    if tuning_method == TuningMethod.distillation:
        kwargs["teacher_model_name"] = args.teacher_args.model_name
        kwargs["teacher_model_class"] = args.teacher_args.model_class
        kwargs["teacher_model_dtype"] = string_to_torch_dtype(args.teacher_args.dtype)
        kwargs["kl_divergence_method"] = args.teacher_args.kl_divergence_method
        kwargs["kl_divergence_weight"] = args.teacher_args.kl_divergence_weight

    cls = _wrapper_class(tuning_method)
    with enable_kernels(args.kernel_args.kernels):
        wrappers = [cls(**kwargs, pipeline_stage_id=stage) for stage in get_pipeline_stage_ids_on_current_rank(num_stages)]
    return ModelContainer(wrappers)


def __getattr__(name: str):
    """The wrapper classes of the other tuning methods and the input broadcast, resolved on first use."""
    import importlib

    lazy = {"ModelWrapperForFinetuning": ".finetuning", "ModelWrapperForDistillation": ".distillation",
            "broadcast_tensor_parallel_input": ".utils"}
    if name in lazy:
        return getattr(importlib.import_module(lazy[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

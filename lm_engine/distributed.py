"""Turns a model container into its distributed-training form.

Parity: lm_engine/distributed.py:140-426 (``wrap_model_container_for_distributed_training``). Where the reference
hands the model to FSDP2 / torch pipelining, this engine installs its own :class:`ShardedTrainingEngine` on every
wrapper (flat sharded storage, explicit collectives) and, for pipeline parallel, its own 1F1B schedule.
"""

from __future__ import annotations

import logging

import torch

from .containers import ModelContainer
from .gradient_checkpointing import apply_gradient_checkpointing
from .optimization.params_group import GROUP_ORDER, get_group_function
from .parallel.engine import ShardedTrainingEngine
from .utils import ProcessGroupManager, log_rank_0, string_to_torch_dtype


def _keep_parameters_gathered(dist_args, wrapper, dtype: torch.dtype) -> bool:
    """Stage 0 and 2 keep every rank's full compute copy (that is what those stages mean). Stage 3 follows
    ``keep_parameters_gathered``; left unset, the gathered weights and the full-size fp32 gradient buffer stay resident
    when they fit comfortably (collectives once per optimizer step instead of per block and micro-step), and the blocks
    are gathered and released one by one when they do not."""
    if dist_args.stage != 3 or ProcessGroupManager.get_sharding_world_size() == 1:
        return True
    if dist_args.keep_parameters_gathered is not None:
        return bool(dist_args.keep_parameters_gathered)
    if not torch.cuda.is_available():
        return True
    params = sum(p.numel() for p in wrapper.parameters() if p.requires_grad)
    width = torch.empty((), dtype=dtype).element_size()
    shard = ProcessGroupManager.get_sharding_world_size()
    resident_bytes = params * (width + 4) + params * 12 // shard
    capacity = torch.cuda.get_device_properties(ProcessGroupManager.get_device()).total_memory
    keep = resident_bytes < 0.6 * capacity
    if not keep:
        log_rank_0(logging.INFO, "stage 3: the gathered weights do not fit next to the activations; blocks are gathered and released one by one")
    return keep


def wrap_model_container_for_distributed_training(args, model_container: ModelContainer):
    dist_args = args.distributed_args
    dtype = string_to_torch_dtype(args.mixed_precision_args.dtype)
    comm_dtype = None if dist_args.communication_dtype is None else string_to_torch_dtype(dist_args.communication_dtype)
    if dist_args.stage not in (0, 2, 3):
        raise ValueError(f"unexpected ZeRO stage ({dist_args.stage})")

    device = ProcessGroupManager.get_device()
    group_of = get_group_function(args.optimizer_args.params_group_method)
    frozen = ("teacher_model.",)

    for wrapper in model_container:
        if dist_args.gradient_checkpointing_method is not None:
            block_names = getattr(wrapper.model, "_no_split_modules", ["Block"])
            apply_gradient_checkpointing(wrapper.model, dist_args.gradient_checkpointing_method,
                                         block_name=block_names[0], **dist_args.gradient_checkpointing_args)
        for name, p in wrapper.named_parameters():
            if name.startswith(frozen):
                p.requires_grad_(False)
        if dist_args.expert_parallel_world_size > 1:
            from .parallel.expert_parallel import set_expert_capacity_factor

            set_expert_capacity_factor(dist_args.expert_capacity_factor)
        engine = ShardedTrainingEngine(
            wrapper,
            resident_parameters=_keep_parameters_gathered(dist_args, wrapper, dtype),
            cpu_offload=dist_args.cpu_offload,
            compute_dtype=dtype,
            zero_stage=dist_args.stage,
            device=device,
            block_class_names=getattr(wrapper.model, "_no_split_modules", None),
            group_of=group_of,
            group_order=GROUP_ORDER,
            communication_dtype=comm_dtype,
            fused_collectives=dist_args.fused_collectives,
            frozen_prefixes=frozen,
            sequence_parallel=dist_args.sequence_parallel,
        )
        wrapper._lm_engine = engine
        wrapper.model._lm_engine = engine
        if hasattr(wrapper, "teacher_model") and wrapper.teacher_model is not None:
            wrapper.teacher_model.to(device)
        log_rank_0(logging.INFO, f"sharded engine: {engine.memory_summary()}")

    if args.mixed_precision_args.dtype == "fp8":
        from .fp8 import FP8Manager

        manager = FP8Manager([w.model for w in model_container], recipe=args.mixed_precision_args.fp8_recipe)
        log_rank_0(logging.INFO, f"fp8 ({manager.recipe}): {manager.converted} linear layers converted (compute dtype of the rest: bf16)")

    pipeline_schedule = None
    if dist_args.num_pipeline_stages > 1:
        from .parallel.pipeline import build_pipeline_schedule

        pipeline_schedule = build_pipeline_schedule(args, model_container)

    if dist_args.torch_compile:
        log_rank_0(logging.WARN, "torch_compile is ignored: hot ops run hand-written kernels, not Inductor output")
    return model_container, pipeline_schedule

"""Finetuning driver: ``python -m lm_engine.finetune --config cfg.yml`` (parity: lm_engine/finetune.py:38-416).

Same skeleton as pretraining with a different loss normalisation: all micro-batches of an accumulation window are
fetched first and ``lm_loss_multiplier = 1 / (number of target tokens in the window on this rank)``, so the step
minimises the mean loss per target token. The dataloader state is part of the checkpoint.
"""

from __future__ import annotations

import logging
from contextlib import nullcontext

import torch

from .arguments import TrainingArgs, get_args
from .checkpointing import ensure_last_checkpoint_is_saved, load_checkpoint_for_training, save_checkpoint
from .containers import LRSchedulerContainer, ModelContainer, OptimizerContainer, log_model_optimizer_container
from .data import custom_iterator, get_next_batch
from .data.finetuning import get_finetuning_dataloader
from .distributed import wrap_model_container_for_distributed_training
from .enums import DatasetSplit, Mode, TuningMethod
from .hf_models import disable_generation_cache
from .kernels import enable_kernels
from .model_wrapper import get_model_container
from .optimization import get_learning_rate, get_optimizer_container, get_scheduler_container
from .pretrain import set_seed
from .train_utils import all_reduce_metrics_tracker, check_device_health, get_torch_profiler, track_metrics
from .utils import (
    ExperimentsTracker,
    MetricsTrackingDict,
    ProcessGroupManager,
    ProgressBar,
    StepTracker,
    init_distributed,
    setup_tf32,
)


def train_step_without_pipeline_parallel(model_container: ModelContainer, optimizer_container: OptimizerContainer,
                                         lr_scheduler_container: LRSchedulerContainer, train_dataloader,
                                         gradient_clipping: float | None, forward_context=nullcontext,
                                         backward_context=nullcontext,
                                         sync_every_gradient_accumulation_step: bool = False) -> MetricsTrackingDict:
    assert len(model_container) == 1
    model = model_container[0]
    engine = model._lm_engine
    ga = StepTracker.get_gradient_accumulation_steps()
    batches = [get_next_batch(train_dataloader) for _ in range(ga)]
    # gradient accumulation is already accounted for: the multiplier spans the whole window
    targets = sum((batch["labels"] != -100).sum() for batch in batches if batch is not None)
    lm_loss_multiplier = 1 / targets
    metrics = MetricsTrackingDict({})
    for batch in batches:
        with forward_context():
            loss_dict = model(batch, lm_loss_multiplier=lm_loss_multiplier)
        with backward_context():
            loss_dict["loss"].backward()
        engine.fold_autograd_grads()
        with torch.inference_mode():
            metrics = metrics + {k: v.detach().float() if isinstance(v, torch.Tensor) else v for k, v in loss_dict.items()}
    grad_norm = engine.optimizer_step(optimizer_container[0], lr_scheduler_container[0], gradient_clipping)
    with torch.inference_mode():
        metrics["grad_norm"] = grad_norm.reshape(()).clone()
        for key in list(metrics.keys()):
            if isinstance(metrics[key], torch.Tensor):
                metrics[key] = metrics[key].item()
        metrics = all_reduce_metrics_tracker(metrics)
    return metrics


@torch.no_grad()
def evaluate(val_dataloader, model_container: ModelContainer, global_step: int, experiments_tracker) -> MetricsTrackingDict | None:
    if val_dataloader is None and not ProcessGroupManager.is_tensor_parallel_enabled():
        return None
    model = model_container[0]
    model_container.eval()
    metrics = MetricsTrackingDict({})
    count = 0
    for batch in val_dataloader:
        targets = (batch["labels"] != -100).sum()
        loss_dict = model(batch, lm_loss_multiplier=1 / targets)
        metrics = metrics + {k: v.detach().float() if isinstance(v, torch.Tensor) else v for k, v in loss_dict.items()}
        count += 1
    if count > 0:
        metrics = metrics / count
    for key in list(metrics.keys()):
        if isinstance(metrics[key], torch.Tensor):
            metrics[key] = metrics[key].item()
    metrics = all_reduce_metrics_tracker(metrics)
    track_metrics(global_step, experiments_tracker, metrics, context="val")
    model_container.train()
    return metrics


def train(args: TrainingArgs, model_container, optimizer_container, lr_scheduler_container, train_dataloader,
          val_dataloader, experiments_tracker, starting_iteration: int = 0) -> None:
    tp = args.training_parameters
    model_container.train()
    if tp.eval_during_training:
        evaluate(val_dataloader, model_container, starting_iteration, experiments_tracker)
    train_iterator = custom_iterator(train_dataloader, infinite=True)
    metrics_tracker = MetricsTrackingDict({})
    profiler = get_torch_profiler(args.logging_args.torch_profiler_trace_path)
    bar = ProgressBar(starting_iteration, tp.num_training_steps)
    with profiler as prof:
        for global_step in range(starting_iteration + 1, tp.num_training_steps + 1):
            loss_dict = train_step_without_pipeline_parallel(
                model_container, optimizer_container, lr_scheduler_container, train_iterator, tp.gradient_clipping,
                sync_every_gradient_accumulation_step=args.distributed_args.sync_every_gradient_accumulation_step)
            metrics_tracker = metrics_tracker + loss_dict
            if prof is not None and hasattr(prof, "step"):
                prof.step()
            bar.update()
            if global_step % args.logging_args.log_interval == 0:
                check_device_health()
                metrics_tracker = metrics_tracker / args.logging_args.log_interval
                metrics_tracker["learning_rate"] = get_learning_rate(model_container, lr_scheduler_container)
                track_metrics(global_step, experiments_tracker, metrics_tracker, context="train")
                metrics_tracker = MetricsTrackingDict({})
            if tp.eval_during_training and (global_step % tp.eval_interval == 0 or global_step == tp.num_training_steps):
                evaluate(val_dataloader, model_container, global_step, experiments_tracker)
            if global_step % args.save_args.save_interval == 0 or global_step == tp.num_training_steps:
                check_device_health()  # never write a checkpoint of a step that ran on partial data
                save_checkpoint(args, model_container, optimizer_container, lr_scheduler_container, train_dataloader,
                                experiments_tracker, global_step)
    ensure_last_checkpoint_is_saved()


def main(argv: list[str] | None = None) -> None:
    mode = Mode.training
    setup_tf32()
    args: TrainingArgs = get_args(mode, argv)
    assert args.tuning_args.tuning_method == TuningMethod.full_finetuning, f"unexpected tuning method ({args.tuning_args.tuning_method})"
    d = args.distributed_args
    assert d.num_pipeline_stages == 1, "pipeline parallel is not supported with finetuning"
    init_distributed(
        tensor_parallel_world_size=d.tensor_parallel_world_size, pipeline_parallel_world_size=d.pipeline_parallel_world_size,
        data_parallel_replication_world_size=d.zero_topology.data_parallel_replication_world_size,
        data_parallel_sharding_world_size=d.zero_topology.data_parallel_sharding_world_size, zero_stage=d.stage,
        timeout_minutes=d.timeout_minutes, use_async_tensor_parallel=d.use_async_tensor_parallel,
        expert_parallel_world_size=d.expert_parallel_world_size)
    StepTracker(micro_batch_size=args.training_parameters.micro_batch_size,
                gradient_accumulation_steps=args.training_parameters.gradient_accumulation_steps)
    set_seed(args.random_args.seed)

    from . import ops

    ops.set_strict(args.kernel_args.strict)
    with enable_kernels(args.kernel_args.kernels):
        model_container = get_model_container(args, mode)
        wrapper = model_container[0]
        train_dataloader = get_finetuning_dataloader(args, DatasetSplit.train, mode, wrapper.tokenizer, wrapper.is_encoder_decoder)
        val_dataloader = None
        if args.training_parameters.eval_during_training:
            val_dataloader = get_finetuning_dataloader(args, DatasetSplit.val, mode, wrapper.tokenizer, wrapper.is_encoder_decoder)
        model_container, _ = wrap_model_container_for_distributed_training(args, model_container)
        optimizer_container = get_optimizer_container(
            optimizer_class_name=args.optimizer_args.class_name, optimizer_class_args=args.optimizer_args.class_args,
            model_container=model_container, params_group_method=args.optimizer_args.params_group_method,
            use_optimizer_with_backward_hook=args.optimizer_args.use_optimizer_with_backward_hook)
        lr_scheduler_container = get_scheduler_container(
            model_container=model_container, optimizer_container=optimizer_container,
            num_warmup_steps=args.lr_scheduler_args.num_warmup_steps, num_constant_steps=args.lr_scheduler_args.num_constant_steps,
            num_decay_steps=args.lr_scheduler_args.num_decay_steps, num_training_steps=args.training_parameters.num_training_steps,
            lr_decay_style=args.lr_scheduler_args.lr_decay_style, lr_decay_factor=args.lr_scheduler_args.lr_decay_factor,
            extra_lr_scheduler_args=args.lr_scheduler_args.extra_lr_scheduler_args,
            use_optimizer_with_backward_hook=args.optimizer_args.use_optimizer_with_backward_hook)
        log_model_optimizer_container(model_container, optimizer_container)

        starting_iteration, tracker_state = 0, None
        if args.load_args is not None:
            starting_iteration, _, tracker_state = load_checkpoint_for_training(
                args, mode, model_container, optimizer_container, lr_scheduler_container, train_dataloader)
        experiments_tracker = ExperimentsTracker(args.logging_args.experiments_tracker_name, args.logging_args.aim_args,
                                                 args.logging_args.wandb_args, checkpoint_metadata=tracker_state)
        experiments_tracker.log_args(args)
        with disable_generation_cache():
            train(args, model_container, optimizer_container, lr_scheduler_container, train_dataloader, val_dataloader,
                  experiments_tracker, starting_iteration)
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()

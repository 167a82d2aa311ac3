"""Pretraining (and distillation) driver: ``python -m lm_engine.pretrain --config cfg.yml``.

Parity: lm_engine/pretrain.py:46-661. YAML -> process groups -> model container -> sharded engine -> optimizer and
schedule -> optional resume -> dataloaders -> loop of (gradient-accumulation micro-steps, clip, step), logging every
``log_interval`` steps, periodic evaluation and checkpointing. Step time is measured on the device (CUDA events) and
reported as the maximum over ranks.
"""

from __future__ import annotations

import logging
import time
from contextlib import nullcontext

import torch
import torch.distributed as dist

from .arguments import DistillationArgs, TrainingArgs, get_args
from .checkpointing import ensure_last_checkpoint_is_saved, load_checkpoint_for_training, save_checkpoint
from .containers import LRSchedulerContainer, ModelContainer, OptimizerContainer, log_model_optimizer_container
from .data import custom_iterator, get_next_batch, get_pretraining_dataloaders
from .distributed import wrap_model_container_for_distributed_training
from .enums import Mode, TuningMethod
from .hf_models import disable_generation_cache
from .kernels import enable_kernels
from .model_wrapper import get_model_container
from .optimization import get_learning_rate, get_optimizer_container, get_scheduler_container
from .train_utils import all_reduce_metrics_tracker, check_device_health, get_model_tflops, get_torch_profiler, track_metrics
from .utils import (
    DeviceTimer,
    ExperimentsTracker,
    MetricsTrackingDict,
    ProcessGroupManager,
    StepTracker,
    init_distributed,
    is_tracking_rank,
    log_rank_0,
    max_over_ranks,
    setup_tf32,
)


def set_seed(seed: int) -> None:
    import random

    import numpy as np

    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def train_step_without_pipeline_parallel(
    model_container: ModelContainer,
    optimizer_container: OptimizerContainer,
    lr_scheduler_container: LRSchedulerContainer,
    train_dataloader,
    gradient_clipping: float | None,
    forward_context=nullcontext,
    backward_context=nullcontext,
    sync_every_gradient_accumulation_step: bool = False,
    lm_loss_multiplier: float = 1,
) -> MetricsTrackingDict:
    """One optimizer step: ``gradient_accumulation_steps`` micro-steps of forward/backward, then reduce, clip, update."""
    assert len(model_container) == 1
    model = model_container[0]
    engine = model._lm_engine
    ga = StepTracker.get_gradient_accumulation_steps()
    metrics = MetricsTrackingDict({})

    for micro_step in range(ga):
        batch = get_next_batch(train_dataloader)
        if micro_step == ga - 1 and hasattr(engine, "arm_early_reduction"):
            engine.arm_early_reduction()  # gradients of a block are reduced as soon as its last backward is done
        with forward_context():
            loss_dict = model(batch, lm_loss_multiplier=lm_loss_multiplier)
        with backward_context():
            (loss_dict["loss"] / ga).backward()
        engine.fold_autograd_grads()
        with torch.inference_mode():
            metrics = metrics + {k: v.detach().float() if isinstance(v, torch.Tensor) else v for k, v in loss_dict.items()}

    grad_norm = engine.optimizer_step(optimizer_container[0], lr_scheduler_container[0], gradient_clipping)
    with torch.inference_mode():
        metrics = metrics / ga
        metrics["grad_norm"] = grad_norm.reshape(())
        for key in list(metrics.keys()):
            if isinstance(metrics[key], torch.Tensor):
                metrics[key] = metrics[key].clone()
    return metrics


def train_step_with_pipeline_parallel(model_container, pipeline_schedule, optimizer_container, lr_scheduler_container,
                                      train_dataloader, gradient_clipping, sequence_length,
                                      lm_loss_multiplier: float | None = None) -> MetricsTrackingDict:
    """One optimizer step through the pipeline schedule; the loss is normalised by ``lm_loss_multiplier``
    (``1 / (micro_batch_size * sequence_length)`` when not given), as in the step without pipeline parallelism."""
    from .parallel.pipeline import pipeline_train_step

    return pipeline_train_step(model_container, pipeline_schedule, optimizer_container, lr_scheduler_container,
                               train_dataloader, gradient_clipping, sequence_length, lm_loss_multiplier=lm_loss_multiplier)


def track_val_metrics(global_step: int, experiments_tracker, metrics_tracker: MetricsTrackingDict, group_name: str | None = None) -> None:
    context = "val" if group_name is None else f"val-{group_name}"
    track_metrics(global_step=global_step, experiments_tracker=experiments_tracker, metrics_tracker=metrics_tracker, context=context)


@torch.no_grad()
def evaluate(val_dataloaders: list, model_container: ModelContainer, global_step: int, experiments_tracker,
             eval_steps: int, group_names: list[str], lm_loss_multiplier: float) -> None:
    if len(val_dataloaders) == 0:
        return
    assert len(model_container) == 1
    model = model_container[0]
    model_container.eval()
    for group_name, loader in zip(group_names, val_dataloaders):
        if loader is None and not ProcessGroupManager.is_tensor_parallel_enabled():
            continue
        metrics = MetricsTrackingDict({})
        for _ in range(eval_steps):
            batch = get_next_batch(loader)
            loss_dict = model(batch, lm_loss_multiplier=lm_loss_multiplier)
            metrics = metrics + {k: v.detach().float() if isinstance(v, torch.Tensor) else v for k, v in loss_dict.items()}
        metrics = metrics / eval_steps
        for key in list(metrics.keys()):
            if isinstance(metrics[key], torch.Tensor):
                metrics[key] = metrics[key].item()
        metrics = all_reduce_metrics_tracker(metrics)
        track_val_metrics(global_step, experiments_tracker, metrics, group_name)
    model_container.train()


def train(args: TrainingArgs, model_container: ModelContainer, pipeline_schedule, optimizer_container, lr_scheduler_container,
          train_dataloader, val_dataloaders: list, test_dataloaders: list, experiments_tracker, starting_iteration: int = 0) -> None:
    tp = args.training_parameters
    num_training_steps = tp.num_training_steps
    ga = tp.gradient_accumulation_steps
    micro_batch_size = tp.micro_batch_size
    sequence_length = args.datasets[0].class_args.get("sequence_length")
    global_batch_size = StepTracker.get_global_batch_size()
    tokens_per_batch = global_batch_size * sequence_length
    lm_loss_multiplier = 1 / (micro_batch_size * sequence_length)
    log_interval = args.logging_args.log_interval
    eval_during_training = tp.eval_during_training
    eval_interval = tp.eval_interval
    eval_steps = args.datasets[0].class_args.get("eval_steps")
    save_interval = args.save_args.save_interval
    val_group_names = _val_group_names(args)

    model_flops = get_model_tflops(
        config=model_container[0].config, batch_size=global_batch_size, sequence_length=sequence_length,
        gradient_checkpointing_method=args.distributed_args.gradient_checkpointing_method,
        gradient_checkpointing_args=args.distributed_args.gradient_checkpointing_args)
    world_size = ProcessGroupManager.get_world_size()

    model_container.train()
    if eval_during_training:
        evaluate(val_dataloaders, model_container, starting_iteration, experiments_tracker, eval_steps, val_group_names, lm_loss_multiplier)

    profiler = get_torch_profiler(args.logging_args.torch_profiler_trace_path)
    profiler_cm = profiler if hasattr(profiler, "__enter__") else nullcontext()
    metrics_tracker = MetricsTrackingDict({})
    timer = DeviceTimer(ProcessGroupManager.get_device())
    timer.start()
    steps_since_log = 0

    with profiler_cm as prof:
        global_step = starting_iteration
        while global_step < num_training_steps:
            global_step += 1
            steps_since_log += 1
            if pipeline_schedule is None:
                loss_dict = train_step_without_pipeline_parallel(
                    model_container, optimizer_container, lr_scheduler_container, train_dataloader, tp.gradient_clipping,
                    sync_every_gradient_accumulation_step=args.distributed_args.sync_every_gradient_accumulation_step,
                    lm_loss_multiplier=lm_loss_multiplier)
            else:
                loss_dict = train_step_with_pipeline_parallel(
                    model_container, pipeline_schedule, optimizer_container, lr_scheduler_container, train_dataloader,
                    tp.gradient_clipping, sequence_length, lm_loss_multiplier=lm_loss_multiplier)
            metrics_tracker = metrics_tracker + loss_dict
            if prof is not None and hasattr(prof, "step"):
                prof.step()

            if global_step % log_interval == 0:
                timer.stop()
                elapsed = max_over_ranks(timer.elapsed_ms() / 1e3)
                step_time = elapsed / steps_since_log
                metrics_tracker = metrics_tracker / steps_since_log
                for key in list(metrics_tracker.keys()):
                    if isinstance(metrics_tracker[key], torch.Tensor):
                        metrics_tracker[key] = metrics_tracker[key].item()
                check_device_health()
                metrics_tracker = all_reduce_metrics_tracker(metrics_tracker)
                metrics_tracker["learning_rate"] = get_learning_rate(model_container, lr_scheduler_container)
                if model_flops:
                    metrics_tracker["FLOPs"] = model_flops / world_size / step_time
                metrics_tracker["billion_tokens_per_day"] = tokens_per_batch * 86400 / step_time / 1e9
                metrics_tracker["tokens_per_second"] = tokens_per_batch / step_time
                metrics_tracker["step_time (sec)"] = step_time
                track_metrics(global_step, experiments_tracker, metrics_tracker, context="train")
                metrics_tracker = MetricsTrackingDict({})
                steps_since_log = 0
                timer.start()

            if eval_during_training and (global_step % eval_interval == 0 or global_step == num_training_steps):
                evaluate(val_dataloaders, model_container, global_step, experiments_tracker, eval_steps, val_group_names, lm_loss_multiplier)

            if global_step % save_interval == 0 or global_step == num_training_steps:
                check_device_health()  # never write a checkpoint of a step that ran on partial data
                save_checkpoint(args, model_container=model_container, optimizer_container=optimizer_container,
                                lr_scheduler_container=lr_scheduler_container, train_dataloader=None,
                                experiments_tracker=experiments_tracker, iteration=global_step,
                                metadata={"consumed_samples": global_step * global_batch_size})
                timer.start()
                steps_since_log = 0

    if eval_during_training and len(test_dataloaders) > 0:
        evaluate(test_dataloaders, model_container, num_training_steps, experiments_tracker, eval_steps, val_group_names, lm_loss_multiplier)
    ensure_last_checkpoint_is_saved()


def _val_group_names(args) -> list[str]:
    class_args = args.datasets[0].class_args
    groups = class_args.get("val_weighted_split_paths")
    if groups:
        names = []
        for group in groups:
            names.extend(group.keys() if isinstance(group, dict) else [str(group)])
        return names
    return [None]


def main(mode: Mode = Mode.training, argv: list[str] | None = None) -> None:
    setup_tf32()
    args: TrainingArgs | DistillationArgs = get_args(mode, argv)
    if mode == Mode.training:
        assert args.tuning_args.tuning_method == TuningMethod.pretraining, f"unexpected tuning method ({args.tuning_args.tuning_method})"
    elif mode == Mode.distillation:
        assert args.tuning_args.tuning_method == TuningMethod.distillation

    d = args.distributed_args
    init_distributed(
        tensor_parallel_world_size=d.tensor_parallel_world_size,
        pipeline_parallel_world_size=d.pipeline_parallel_world_size,
        data_parallel_replication_world_size=d.zero_topology.data_parallel_replication_world_size,
        data_parallel_sharding_world_size=d.zero_topology.data_parallel_sharding_world_size,
        zero_stage=d.stage,
        timeout_minutes=d.timeout_minutes,
        use_async_tensor_parallel=d.use_async_tensor_parallel,
        expert_parallel_world_size=d.expert_parallel_world_size,
    )
    StepTracker(micro_batch_size=args.training_parameters.micro_batch_size,
                gradient_accumulation_steps=args.training_parameters.gradient_accumulation_steps)
    set_seed(args.random_args.seed)

    from . import ops

    ops.set_strict(args.kernel_args.strict)
    with enable_kernels(args.kernel_args.kernels):
        model_container = get_model_container(args, mode)
        model_container, pipeline_schedule = wrap_model_container_for_distributed_training(args, model_container)
        optimizer_container = get_optimizer_container(
            optimizer_class_name=args.optimizer_args.class_name, optimizer_class_args=args.optimizer_args.class_args,
            model_container=model_container, params_group_method=args.optimizer_args.params_group_method,
            use_optimizer_with_backward_hook=args.optimizer_args.use_optimizer_with_backward_hook)
        lr_scheduler_container = get_scheduler_container(
            model_container=model_container, optimizer_container=optimizer_container,
            num_warmup_steps=args.lr_scheduler_args.num_warmup_steps,
            num_constant_steps=args.lr_scheduler_args.num_constant_steps,
            num_decay_steps=args.lr_scheduler_args.num_decay_steps,
            num_training_steps=args.training_parameters.num_training_steps,
            lr_decay_style=args.lr_scheduler_args.lr_decay_style, lr_decay_factor=args.lr_scheduler_args.lr_decay_factor,
            extra_lr_scheduler_args=args.lr_scheduler_args.extra_lr_scheduler_args,
            use_optimizer_with_backward_hook=args.optimizer_args.use_optimizer_with_backward_hook)
        log_model_optimizer_container(model_container, optimizer_container)

        starting_iteration = 0
        metadata = None
        experiments_tracker_state = None
        if args.load_args is not None:
            starting_iteration, metadata, experiments_tracker_state = load_checkpoint_for_training(
                args, mode, model_container, optimizer_container, lr_scheduler_container, None)
            if metadata is not None and args.load_args.load_dataloader_state:
                consumed = metadata.get("consumed_samples", 0)
            else:
                consumed = 0
        else:
            consumed = 0

        train_dataloader, val_dataloaders, test_dataloaders = get_pretraining_dataloaders(
            args, model_container[0].tokenizer, consumed)
        experiments_tracker = ExperimentsTracker(args.logging_args.experiments_tracker_name, args.logging_args.aim_args,
                                                 args.logging_args.wandb_args, checkpoint_metadata=experiments_tracker_state)
        experiments_tracker.log_args(args)

        with disable_generation_cache():
            train(args, model_container, pipeline_schedule, optimizer_container, lr_scheduler_container,
                  train_dataloader, val_dataloaders, test_dataloaders, experiments_tracker, starting_iteration)
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()

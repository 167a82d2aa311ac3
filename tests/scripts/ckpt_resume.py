"""Phase "save": train 3 steps, checkpoint, train 2 more and record their losses. Phase "resume": load the checkpoint
and train the 2 steps again. Phase "unshard" (one process): rebuild the single-device model from the checkpoint and write its
weights. Usage: [torchrun ...] ckpt_resume.py <phase> <save_dir> <out.json> [async|sync] [expert parallel size]
[tensor parallel size]"""

import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from tiny_pretrain import tiny_config

from lm_engine.arguments import args_from_dict
from lm_engine.checkpointing import ensure_last_checkpoint_is_saved, load_checkpoint_for_training, save_checkpoint
from lm_engine.data import get_pretraining_dataloaders
from lm_engine.distributed import wrap_model_container_for_distributed_training
from lm_engine.enums import Mode
from lm_engine.model_wrapper import get_model_container
from lm_engine.optimization import get_optimizer_container, get_scheduler_container
from lm_engine.pretrain import set_seed, train_step_without_pipeline_parallel
from lm_engine.train_utils import all_reduce_metrics_tracker
from lm_engine.utils import ProcessGroupManager, StepTracker, init_distributed


def main() -> None:
    phase, save_dir, out_path = sys.argv[1], sys.argv[2], sys.argv[3]
    use_async = len(sys.argv) > 4 and sys.argv[4] == "async"
    world = int(os.environ.get("WORLD_SIZE", 1))
    ep = int(sys.argv[5]) if len(sys.argv) > 5 else 0
    tp = int(sys.argv[6]) if len(sys.argv) > 6 else 1
    if phase == "unshard":
        from lm_engine.arguments import UnshardingArgs
        from lm_engine.checkpointing import load_checkpoint_for_inference

        args = UnshardingArgs(load_args=dict(load_path=save_dir), unsharded_path=os.path.join(save_dir, "unsharded"))
        _, _, state = load_checkpoint_for_inference(args, Mode.unsharding, use_meta=False)
        torch.save({k: v.float() for k, v in state.items()}, out_path)
        return
    config = tiny_config(8 // (world // tp), 5, ep=ep, tp=tp)
    config["save_args"] = dict(save_path=save_dir, save_interval=3, async_checkpointing=use_async)
    if phase == "resume":
        config["load_args"] = dict(load_path=save_dir)
    args = args_from_dict(Mode.training, config)
    init_distributed(zero_stage=3, expert_parallel_world_size=max(ep, 1), tensor_parallel_world_size=tp)
    StepTracker(args.training_parameters.micro_batch_size, 1)
    set_seed(42 if phase == "save" else 7)  # a resumed run must not depend on its own seed
    container = get_model_container(args, Mode.training)
    container, _ = wrap_model_container_for_distributed_training(args, container)
    optimizers = get_optimizer_container("TorchAdamW", args.optimizer_args.class_args, container)
    schedulers = get_scheduler_container(container, optimizers, 2, 0, None, 5, args.lr_scheduler_args.lr_decay_style, 0.1, {})
    container.train()
    multiplier = 1 / (args.training_parameters.micro_batch_size * 128)

    start = 0
    consumed = 0
    if phase == "resume":
        start, metadata, _ = load_checkpoint_for_training(args, Mode.training, container, optimizers, schedulers, None)
        consumed = metadata["consumed_samples"]
    loader, _, _ = get_pretraining_dataloaders(args, None, consumed)

    curve = []
    for step in range(start + 1, 6):
        metrics = train_step_without_pipeline_parallel(container, optimizers, schedulers, loader, 1.0, lm_loss_multiplier=multiplier)
        for key in list(metrics.keys()):
            metrics[key] = float(metrics[key])
        metrics = all_reduce_metrics_tracker(metrics)
        if step > 3:
            curve.append(metrics["loss"])
        if phase == "save" and step == 3:
            save_checkpoint(args, container, optimizers, schedulers, None, None, step, metadata={"consumed_samples": step * 8})
    ensure_last_checkpoint_is_saved()
    if ProcessGroupManager.get_global_rank() == 0:
        with open(out_path, "w") as handle:
            json.dump({"losses": curve, "lr": schedulers[0].get_last_lr()[0]}, handle)
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()

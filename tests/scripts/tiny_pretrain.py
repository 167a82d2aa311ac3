"""Runs N optimizer steps of the tiny gpt_base pretraining config on CPU (any world size) and writes the loss curve.

Usage: [torchrun ...] tiny_pretrain.py <output.json> <global_batch> <steps> [zero stage] [tensor parallel size] [sequence parallel 0/1]
"""

import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from lm_engine.arguments import args_from_dict
from lm_engine.data import get_pretraining_dataloaders
from lm_engine.distributed import wrap_model_container_for_distributed_training
from lm_engine.enums import Mode
from lm_engine.model_wrapper import get_model_container
from lm_engine.optimization import get_optimizer_container, get_scheduler_container
from lm_engine.pretrain import set_seed, train_step_without_pipeline_parallel
from lm_engine.train_utils import all_reduce_metrics_tracker
from lm_engine.utils import ProcessGroupManager, StepTracker, init_distributed


def tiny_config(micro_batch_size: int, steps: int, ga: int = 1, stage: int = 3, tp: int = 1, sp: bool = False) -> dict:
    layer_attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=4, add_bias=False)
    layer_mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=256, add_bias=False)
    return dict(
        datasets=[dict(class_name="SyntheticDataset", data_name="synthetic", class_args=dict(sequence_length=128, seed=7))],
        model_args=dict(
            model_class="AutoModelForCausalLM",
            use_padding_free_transformer=False,
            pretrained_config=dict(
                model_type="gpt_base", vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope",
                rope_theta=10000, normalization_function="rmsnorm", layer_norm_epsilon=1e-5, tie_word_embeddings=False,
                max_position_embeddings=128, initializer_range=0.02,
                sequence_mixer_blocks=[layer_attn, layer_attn], mlp_blocks=[layer_mlp, layer_mlp]),
        ),
        tuning_args=dict(tuning_method="pretraining"),
        save_args=dict(save_path="/tmp/unused", save_interval=10**9),
        training_parameters=dict(num_training_steps=steps, micro_batch_size=micro_batch_size,
                                 gradient_accumulation_steps=ga, eval_during_training=False, gradient_clipping=1.0),
        optimizer_args=dict(class_name="TorchAdamW", class_args=dict(lr=3e-4, weight_decay=0.1, betas=[0.9, 0.95], eps=1e-10)),
        lr_scheduler_args=dict(lr_decay_style="cosine", num_warmup_steps=2),
        mixed_precision_args=dict(dtype="fp32"),
        distributed_args=dict(stage=stage, tensor_parallel_world_size=tp, sequence_parallel=sp),
    )


def main() -> None:
    out_path, global_batch, steps = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    stage = int(sys.argv[4]) if len(sys.argv) > 4 else 3
    tp = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    sp = bool(int(sys.argv[6])) if len(sys.argv) > 6 else False
    world = int(os.environ.get("WORLD_SIZE", 1))
    args = args_from_dict(Mode.training, tiny_config(global_batch // (world // tp), steps, stage=stage, tp=tp, sp=sp))
    init_distributed(zero_stage=stage, tensor_parallel_world_size=tp)
    StepTracker(args.training_parameters.micro_batch_size, 1)
    set_seed(42)
    container = get_model_container(args, Mode.training)
    container, _ = wrap_model_container_for_distributed_training(args, container)
    optimizers = get_optimizer_container("TorchAdamW", args.optimizer_args.class_args, container)
    schedulers = get_scheduler_container(container, optimizers, 2, 0, None, steps, args.lr_scheduler_args.lr_decay_style, 0.1, {})
    loader, _, _ = get_pretraining_dataloaders(args, None, 0)
    container.train()
    multiplier = 1 / (args.training_parameters.micro_batch_size * 128)
    curve = []
    for _ in range(steps):
        metrics = train_step_without_pipeline_parallel(container, optimizers, schedulers, loader, 1.0, lm_loss_multiplier=multiplier)
        for key in list(metrics.keys()):
            metrics[key] = float(metrics[key])
        grad_norm = metrics["grad_norm"]
        metrics = all_reduce_metrics_tracker(metrics)
        curve.append({"loss": metrics["loss"], "grad_norm": grad_norm})
    if ProcessGroupManager.get_global_rank() == 0:
        with open(out_path, "w") as handle:
            json.dump(curve, handle)
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()

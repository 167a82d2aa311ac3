"""Runs N optimizer steps of the tiny gpt_base pretraining config on CPU (any world size) and writes the loss curve.

Usage: [torchrun ...] tiny_pretrain.py <output.json> <global_batch> <steps> [zero stage] [tensor parallel size] [sequence parallel 0/1]
       [pipeline parallel size] [pipeline stages] [schedule] [gradient accumulation steps] [sync|nosync] [expert parallel size:
       the model then has mixture-of-experts MLPs]
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


def tiny_config(micro_batch_size: int, steps: int, ga: int = 1, stage: int = 3, tp: int = 1, sp: bool = False, pp: int = 1,
                stages: int = 1, schedule: str | None = None, ep: int = 0) -> dict:
    layer_attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=4, add_bias=False)
    layer_mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=256, add_bias=False)
    if ep > 0:
        layer_mlp = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=64, add_bias=False, num_experts=4, num_experts_per_tok=2)
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
        distributed_args=dict(stage=stage, tensor_parallel_world_size=tp, sequence_parallel=sp, pipeline_parallel_world_size=pp,
                              num_pipeline_stages=stages, pipeline_parallel_schedule=schedule, **({"expert_parallel_world_size": ep} if ep > 1 else {}),
                              **({"keep_parameters_gathered": False} if os.environ.get("TINY_SHARDED_PARAMETERS") == "1" else {}),
                              **({"cpu_offload": True} if os.environ.get("TINY_CPU_OFFLOAD") == "1" else {})),
    )


def main() -> None:
    out_path, global_batch, steps = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    stage = int(sys.argv[4]) if len(sys.argv) > 4 else 3
    tp = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    sp = bool(int(sys.argv[6])) if len(sys.argv) > 6 else False
    pp = int(sys.argv[7]) if len(sys.argv) > 7 else 1
    stages = int(sys.argv[8]) if len(sys.argv) > 8 else 1
    schedule = sys.argv[9] if len(sys.argv) > 9 else None
    ga = int(sys.argv[10]) if len(sys.argv) > 10 else 1
    ep = int(sys.argv[12]) if len(sys.argv) > 12 else 0
    world = int(os.environ.get("WORLD_SIZE", 1))
    micro = global_batch // (world // (tp * pp)) // ga
    args = args_from_dict(Mode.training, tiny_config(micro, steps, ga=ga, stage=stage, tp=tp, sp=sp, pp=pp, stages=stages, schedule=schedule, ep=ep))
    init_distributed(zero_stage=stage, tensor_parallel_world_size=tp, pipeline_parallel_world_size=pp, expert_parallel_world_size=max(ep, 1))
    StepTracker(args.training_parameters.micro_batch_size, ga)
    set_seed(42)
    container = get_model_container(args, Mode.training)
    container, pipeline_schedule = wrap_model_container_for_distributed_training(args, container)
    if len(sys.argv) > 11 and sys.argv[11] == "sync":
        # every layout starts from the weights of one single-device model, cut to what each rank holds
        from lm_engine.hf_models import GPTBaseForCausalLM
        from lm_engine.hf_models.tp_weights import shard_state_dict

        from lm_engine.utils import parallel as parallel_state

        saved_ep = parallel_state._State.ep_world_size
        parallel_state._State.ep_world_size = 1  # the reference holds all experts
        torch.manual_seed(123)
        reference = GPTBaseForCausalLM(container[0].config)
        parallel_state._State.ep_world_size = saved_ep
        full_state = reference.state_dict()
        for wrapper in container:
            if ep > 1:
                per = 4 // ep
                lo = ProcessGroupManager.get_expert_parallel_rank() * per
                part = {k: (v[lo : lo + per] if ".mlp_block.c_fc." in k or ".mlp_block.c_proj." in k else v) for k, v in full_state.items()}
            elif tp > 1 or pp > 1:
                part = shard_state_dict(wrapper.config, full_state, ProcessGroupManager.get_tensor_parallel_rank(), tp, stages,
                                        wrapper.pipeline_stage_id)
            else:
                part = full_state
            wrapper._lm_engine.load_full_state_dict({f"model.{k}": v for k, v in part.items()})
    optimizers = get_optimizer_container("TorchAdamW", args.optimizer_args.class_args, container)
    schedulers = get_scheduler_container(container, optimizers, 2, 0, None, steps, args.lr_scheduler_args.lr_decay_style, 0.1, {})
    loader, _, _ = get_pretraining_dataloaders(args, None, 0)
    container.train()
    multiplier = 1 / (args.training_parameters.micro_batch_size * 128)
    curve = []
    for _ in range(steps):
        if pipeline_schedule is None:
            metrics = train_step_without_pipeline_parallel(container, optimizers, schedulers, loader, 1.0, lm_loss_multiplier=multiplier)
        else:
            # the entry point's own call: the loss normalisation is derived from micro-batch size and sequence length
            from lm_engine.pretrain import train_step_with_pipeline_parallel

            metrics = train_step_with_pipeline_parallel(container, pipeline_schedule, optimizers, schedulers, loader, 1.0, 128)
        for key in list(metrics.keys()):
            metrics[key] = float(metrics[key])
        grad_norm = metrics["grad_norm"]
        has_loss = "loss" in list(metrics.keys())
        if has_loss:
            metrics = all_reduce_metrics_tracker(metrics)
        curve.append({"loss": metrics["loss"] if has_loss else None, "grad_norm": grad_norm})
    from lm_engine.utils import is_tracking_rank

    if os.environ.get("TINY_REPORT_STORAGE") == "1" and curve:
        # where the fp32 master shards and the optimizer's moments live (the cpu_offload test looks at this)
        engine = getattr(container[0], "_lm_engine", None)
        if engine is not None:
            segment = engine.units[0].segments[0]
            state = optimizers[0].state.get(segment.master, {})
            curve[-1]["master_device"] = str(engine.units[0].master.device)
            curve[-1]["optimizer_state_device"] = str(state["exp_avg"].device) if "exp_avg" in state else None
    if is_tracking_rank():
        with open(out_path, "w") as handle:
            json.dump(curve, handle)
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()

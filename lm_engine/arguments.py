"""YAML schema of every entry point.

One YAML file per run; each top-level key is a strict pydantic section (unknown keys are errors). The section and
field names follow lm_engine/arguments.py:32-526 of the reference so existing configs keep working. Fields that
exist only here: ``distributed_args.expert_parallel_world_size``, ``distributed_args.fused_collectives``,
``distributed_args.keep_parameters_gathered``, ``mixed_precision_args.fp8_recipe`` and ``kernel_args.strict``.
"""

from __future__ import annotations

import logging
from argparse import ArgumentParser
from typing import Any

import transformers
from pydantic import Field

from .defaults import INPUT_FORMAT, OUTPUT_FORMAT
from .enums import (
    ExperimentsTrackerName,
    GradientCheckpointingMethod,
    Kernel,
    KLDivergenceMethod,
    LossMask,
    LRDecaySchedule,
    Mode,
    ParamsGroupMethod,
    TuningMethod,
)
from .utils import BaseArgs, load_yaml, log_environment, log_rank_0, normalize_dtype_string, run_rank_n, set_logger

_MODEL_CLASSES = ("AutoModelForCausalLM", "AutoModelForSeq2SeqLM")


def _require(section: str, **fields: Any) -> None:
    missing = [name for name, value in fields.items() if value is None]
    if missing:
        raise ValueError(f"{section}: missing required field(s) {', '.join(missing)}")


def _resolve_model_class(name: str):
    if name not in _MODEL_CLASSES:
        raise ValueError(f"unexpected model_class ({name}); expected one of {_MODEL_CLASSES}")
    return getattr(transformers, name)


class RandomArgs(BaseArgs):
    seed: int = 42


class TokenizerArgs(BaseArgs):
    tokenizer_name: str | None = None
    additional_special_tokens: list[str] | None = None


class ModelArgs(BaseArgs):
    # exactly one of model_name (weights are loaded) / pretrained_config (random init) must be given
    model_name: str | None = None
    pretrained_config: dict | None = None
    model_class: Any = None
    trust_remote_code: bool = False
    use_padding_free_transformer: bool = False
    # build on the meta device and materialise shards only
    efficient_initialization: bool = False
    # pretraining: restart attention / positions at document boundaries (EOS tokens)
    reset_attention_mask: bool = False
    reset_position_ids: bool = False

    def model_post_init(self, __context: Any) -> None:
        _require("model_args", model_class=self.model_class)
        if self.model_name is None:
            _require("model_args", pretrained_config=self.pretrained_config)
        elif self.pretrained_config is not None:
            raise ValueError("model_args: pretrained_config can't be combined with model_name")
        if isinstance(self.model_class, str):
            self.model_class = _resolve_model_class(self.model_class)


class TuningArgs(BaseArgs):
    tuning_method: TuningMethod = None

    def model_post_init(self, __context: Any) -> None:
        _require("tuning_args", tuning_method=self.tuning_method)


class TrainingParameters(BaseArgs):
    ignore_sampling_proportion_for_validation: bool = False
    num_training_steps: int | None = None
    gradient_accumulation_steps: int = 1
    eval_interval: int | None = None
    micro_batch_size: int = None
    eval_during_training: bool = True
    loss_mask: LossMask = LossMask.output_only
    gradient_clipping: float | None = 1

    def model_post_init(self, __context: Any) -> None:
        _require(
            "training_parameters", num_training_steps=self.num_training_steps, micro_batch_size=self.micro_batch_size
        )
        if self.eval_during_training:
            _require("training_parameters", eval_interval=self.eval_interval)


class SaveArgs(BaseArgs):
    save_path: str = None
    save_interval: int = None
    save_optimizer: bool = True
    async_checkpointing: bool = False

    def model_post_init(self, __context: Any) -> None:
        _require("save_args", save_path=self.save_path, save_interval=self.save_interval)


class LoadArgs(BaseArgs):
    load_path: str = None
    iteration: int | None = None
    load_optimizer: bool = True
    load_lr_scheduler: bool = True
    load_rng_state: bool = True
    load_dataloader_state: bool = True
    load_experiments_tracker_state: bool = True
    load_starting_iteration: bool = True
    # rebuild the schedule at the resumed step when the scheduler state itself is not loaded
    resume_learning_rate: bool = True

    def model_post_init(self, __context: Any) -> None:
        _require("load_args", load_path=self.load_path)
        if not self.load_optimizer and self.load_lr_scheduler:
            raise ValueError("load_args: loading the lr scheduler without the optimizer makes no sense")
        if self.load_lr_scheduler and not self.resume_learning_rate:
            raise ValueError("load_args: resume_learning_rate must stay True when the lr scheduler is reloaded")


class DatasetArgs(BaseArgs):
    class_name: str = None
    class_args: dict = {}
    data_name: str = None
    input_format: str = INPUT_FORMAT
    output_format: str = OUTPUT_FORMAT
    data_sampling_ratio: int | None = None
    max_input_tokens: int | None = None
    max_output_tokens: int | None = None

    def model_post_init(self, __context: Any) -> None:
        _require("datasets[]", class_name=self.class_name, data_name=self.data_name)
        if self.data_sampling_ratio is not None and self.data_sampling_ratio <= 0:
            raise ValueError("datasets[]: data_sampling_ratio must be a positive integer")


class OptimizerArgs(BaseArgs):
    class_name: str = "TorchAdamW"
    params_group_method: ParamsGroupMethod | None = None
    use_optimizer_with_backward_hook: bool = False
    class_args: dict = Field(default_factory=lambda: {"lr": 1e-5, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10})

    def model_post_init(self, __context: Any) -> None:
        _require("optimizer_args", class_name=self.class_name)


class LRSchedulerArgs(BaseArgs):
    num_warmup_steps: int = 200
    num_constant_steps: int = 0
    # None: every step after warmup + constant is a decay step
    num_decay_steps: int | None = None
    lr_decay_style: LRDecaySchedule = LRDecaySchedule.cosine
    # min_lr / max_lr
    lr_decay_factor: float = 0.1
    # coefficients of the power schedule: {"a": ..., "b": ..., "c": ...}
    extra_lr_scheduler_args: dict = {}


class MixedPrecisionArgs(BaseArgs):
    dtype: str = "fp32"
    scaling_type_input: str = "dynamic"
    scaling_type_weight: str = "dynamic"
    scaling_type_grad_output: str = "dynamic"
    # "tensorwise" (one scale per tensor) or "mxfp8" (e4m3 payload, one UE8M0 scale per 32 elements along K)
    fp8_recipe: str = "tensorwise"

    def model_post_init(self, __context: Any) -> None:
        self.dtype = normalize_dtype_string(self.dtype)
        if self.fp8_recipe not in ("tensorwise", "mxfp8"):
            raise ValueError(f"mixed_precision_args: unknown fp8_recipe ({self.fp8_recipe})")


class ZeroTopologyArgs(BaseArgs):
    data_parallel_replication_world_size: int | None = None
    data_parallel_sharding_world_size: int | None = None

    def model_post_init(self, __context: Any) -> None:
        a, b = self.data_parallel_replication_world_size, self.data_parallel_sharding_world_size
        if (a is None) != (b is None):
            raise ValueError("zero_topology: give both replication and sharding world sizes, or neither")


class DistributedArgs(BaseArgs):
    # ZeRO stage: 0 (replicate), 2 (shard grads + optimizer), 3 (shard params too)
    stage: int = 3
    # fp32 master shards, optimizer state and a staging copy of the gradient shard in pinned host memory; the optimizer
    # step runs on the CPU (12 bytes per parameter / N leave the device, at the price of two PCIe transfers per step)
    cpu_offload: bool = False
    gradient_checkpointing_method: GradientCheckpointingMethod | None = None
    gradient_checkpointing_args: dict = {}
    zero_topology: ZeroTopologyArgs = ZeroTopologyArgs()
    communication_dtype: str | None = None
    torch_compile: bool = False
    dispatching_dataloader: bool = False
    tensor_parallel_world_size: int = 1
    sequence_parallel: bool = False
    pipeline_parallel_world_size: int = 1
    timeout_minutes: int | None = None
    fsdp_algorithm: int = 2
    sync_every_gradient_accumulation_step: bool = False
    num_pipeline_stages: int = 1
    pipeline_parallel_schedule: str | None = None
    use_async_tensor_parallel: bool = False
    # ---- additions
    expert_parallel_world_size: int = 1
    # True: collectives are issued from this engine's own peer-memory kernels; False: NCCL baseline path
    fused_collectives: bool = True
    # expert parallelism: None = dropless, row buffers sized per layer for the fullest rank (one small device-to-host
    # read per MoE layer); a factor >= 1 = static buffers of that multiple of a rank's balanced share, no host read,
    # entries beyond it are dropped and counted.
    expert_capacity_factor: float | None = None
    # ZeRO-3 only. None: keep the gathered bf16 weights for a whole optimizer step when they fit in memory,
    # otherwise gather per block; True / False force one or the other.
    keep_parameters_gathered: bool | None = None

    def model_post_init(self, __context: Any) -> None:
        if self.communication_dtype is not None:
            self.communication_dtype = normalize_dtype_string(self.communication_dtype)
        if self.stage not in (0, 2, 3):
            raise ValueError("distributed_args: stage must be 0, 2 or 3")
        if self.sequence_parallel and self.tensor_parallel_world_size <= 1:
            raise ValueError("distributed_args: sequence_parallel needs tensor_parallel_world_size > 1")
        if self.tensor_parallel_world_size > 1 and self.fsdp_algorithm != 2:
            raise ValueError("distributed_args: tensor parallel needs fsdp_algorithm 2")
        if self.use_async_tensor_parallel and not self.sequence_parallel:
            raise ValueError("distributed_args: async tensor parallel needs sequence_parallel")
        if self.num_pipeline_stages % self.pipeline_parallel_world_size != 0:
            raise ValueError("distributed_args: num_pipeline_stages must be a multiple of pipeline_parallel_world_size")
        if self.num_pipeline_stages > 1:
            _require("distributed_args", pipeline_parallel_schedule=self.pipeline_parallel_schedule)


class AimArgs(BaseArgs):
    repo: str = None
    experiment: str = None

    def model_post_init(self, __context: Any) -> None:
        _require("aim_args", repo=self.repo, experiment=self.experiment)


class WandBArgs(BaseArgs):
    project: str = None
    name: str = None
    entity: str | None = None

    def model_post_init(self, __context: Any) -> None:
        _require("wandb_args", project=self.project, name=self.name)


class LoggingArgs(BaseArgs):
    logging_level: str = "INFO"
    log_interval: int = 10
    aim_args: AimArgs | None = None
    wandb_args: WandBArgs | None = None
    experiments_tracker_name: ExperimentsTrackerName | None = None
    use_colored_logs: bool = False
    # giving a path turns the torch profiler on (one traced step on rank 0)
    torch_profiler_trace_path: str | None = None

    def model_post_init(self, __context: Any) -> None:
        if self.experiments_tracker_name == ExperimentsTrackerName.aim:
            _require("logging_args", aim_args=self.aim_args)
        elif self.experiments_tracker_name == ExperimentsTrackerName.wandb:
            _require("logging_args", wandb_args=self.wandb_args)


class KernelArgs(BaseArgs):
    kernels: list[Kernel] = []
    # raise when an op would run its PyTorch restatement on CUDA bf16 tensors instead of the sm_100a kernel
    # (without it such a site is counted and logged once; see lm_engine.ops.fallback_counts)
    strict: bool = False


class TeacherArgs(BaseArgs):
    model_class: Any = None
    model_name: str | None = None
    dtype: str = "fp32"
    kl_divergence_method: KLDivergenceMethod = None
    kl_divergence_weight: float = 1

    def model_post_init(self, __context: Any) -> None:
        self.dtype = normalize_dtype_string(self.dtype)
        _require("teacher_args", model_class=self.model_class, kl_divergence_method=self.kl_divergence_method)
        if isinstance(self.model_class, str):
            self.model_class = _resolve_model_class(self.model_class)


def _validate_datasets(datasets: list[DatasetArgs]) -> None:
    if len(datasets) == 0:
        raise ValueError("datasets cannot be an empty list")
    names = [d.data_name for d in datasets]
    if len(set(names)) != len(names):
        raise ValueError("data_name must be unique across datasets")


class TrainingArgs(BaseArgs):
    random_args: RandomArgs = RandomArgs()
    tokenizer_args: TokenizerArgs = TokenizerArgs()
    model_args: ModelArgs = None
    tuning_args: TuningArgs = None
    optimizer_args: OptimizerArgs = OptimizerArgs()
    lr_scheduler_args: LRSchedulerArgs = LRSchedulerArgs()
    datasets: list[DatasetArgs] = []
    save_args: SaveArgs = None
    load_args: LoadArgs | None = None
    training_parameters: TrainingParameters | None = None
    logging_args: LoggingArgs = LoggingArgs()
    mixed_precision_args: MixedPrecisionArgs = MixedPrecisionArgs()
    distributed_args: DistributedArgs = DistributedArgs()
    kernel_args: KernelArgs = KernelArgs()

    def model_post_init(self, __context: Any) -> None:
        _require("training args", model_args=self.model_args, tuning_args=self.tuning_args, save_args=self.save_args)
        _validate_datasets(self.datasets)
        if self.distributed_args.num_pipeline_stages > 1 and self.training_parameters.eval_during_training:
            raise NotImplementedError("evaluation is not supported with pipeline parallel")
        if self.optimizer_args.use_optimizer_with_backward_hook:
            if self.training_parameters.gradient_accumulation_steps != 1:
                raise ValueError("optimizer in backward hook needs gradient_accumulation_steps == 1")
            if self.training_parameters.gradient_clipping is not None:
                raise ValueError("optimizer in backward hook can't clip gradients")


class GenerationParameters(BaseArgs):
    batch_size: int = None
    do_sample: bool | None = None
    max_new_tokens: int = None
    temperature: float | None = None
    top_k: int | None = None
    top_p: float | None = None

    def model_post_init(self, __context: Any) -> None:
        _require("generation_parameters", batch_size=self.batch_size, max_new_tokens=self.max_new_tokens)


class InferenceArgs(BaseArgs):
    random_args: RandomArgs = RandomArgs()
    tokenizer_args: TokenizerArgs = TokenizerArgs()
    model_args: ModelArgs | None = None
    datasets: list[DatasetArgs] = []
    load_args: LoadArgs | None = None
    generation_parameters: GenerationParameters = None
    mixed_precision_args: MixedPrecisionArgs = MixedPrecisionArgs()
    logging_args: LoggingArgs = LoggingArgs()
    output_dir: str = None
    kernel_args: KernelArgs = KernelArgs()

    def model_post_init(self, __context: Any) -> None:
        _require("inference args", generation_parameters=self.generation_parameters, output_dir=self.output_dir)
        if (self.load_args is None) == (self.model_args is None):
            raise ValueError("inference args: give exactly one of model_args / load_args")
        _validate_datasets(self.datasets)


class UnshardingArgs(BaseArgs):
    load_args: LoadArgs = None
    unsharded_path: str = None
    mixed_precision_args: MixedPrecisionArgs = MixedPrecisionArgs()
    logging_args: LoggingArgs = LoggingArgs()
    kernel_args: KernelArgs = KernelArgs()

    def model_post_init(self, __context: Any) -> None:
        _require("unsharding args", load_args=self.load_args, unsharded_path=self.unsharded_path)


class DistillationArgs(TrainingArgs):
    teacher_args: TeacherArgs = None

    def model_post_init(self, __context: Any) -> None:
        _require("distillation args", teacher_args=self.teacher_args)
        super().model_post_init(__context)


_ARGS_OF_MODE = {
    Mode.training: TrainingArgs,
    Mode.inference: InferenceArgs,
    Mode.unsharding: UnshardingArgs,
    Mode.distillation: DistillationArgs,
}


def args_from_dict(mode: Mode, config: dict) -> TrainingArgs | InferenceArgs | UnshardingArgs | DistillationArgs:
    # top-level keys that start with an underscore only hold YAML anchors (shared layer descriptions)
    return _ARGS_OF_MODE[mode](**{k: v for k, v in config.items() if not k.startswith("_")})


def get_args(mode: Mode, argv: list[str] | None = None):
    """Parse ``--config path.yml`` into the argument tree of ``mode`` and log it."""
    parser = ArgumentParser()
    parser.add_argument("--config", type=str, required=True, help="path of the YAML config")
    cli = parser.parse_args(argv)

    args = args_from_dict(mode, load_yaml(cli.config))
    set_logger(args.logging_args.logging_level, colored_log=args.logging_args.use_colored_logs)
    log_args(args)
    log_environment()
    return args


def _render(node: Any, indent: int) -> list[str]:
    pad = " " * indent
    if isinstance(node, BaseArgs):
        node = {name: getattr(node, name) for name in type(node).model_fields}
    lines: list[str] = []
    for key in sorted(node, key=str.lower):
        value = node[key]
        dots = "." * max(2, 48 - len(str(key)) - indent)
        if isinstance(value, (BaseArgs, dict)) and (isinstance(value, BaseArgs) or len(value) > 0):
            lines.append(f"{pad}{key}:")
            lines.extend(_render(value, indent + 4))
        elif isinstance(value, list) and value and all(isinstance(v, (BaseArgs, dict)) for v in value):
            lines.append(f"{pad}{key}:")
            for i, item in enumerate(value):
                if i > 0:
                    lines.append(" " * (indent + 4) + "*" * max(4, 44 - indent))
                lines.extend(_render(item, indent + 4))
        else:
            lines.append(f"{pad}{key} {dots} {value}")
    return lines


@run_rank_n
def log_args(args: BaseArgs) -> None:
    log_rank_0(logging.INFO, "------------------------ arguments ------------------------")
    for line in _render(args, 0):
        log_rank_0(logging.INFO, line)
    log_rank_0(logging.INFO, "-------------------- end of arguments ---------------------")

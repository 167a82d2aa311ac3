"""Enumerations that appear as values in YAML configs (parity: lm_engine/enums.py:8-89)."""

from __future__ import annotations

from enum import Enum


def _enum(name: str, values: list[str], doc: str) -> type[Enum]:
    cls = Enum(name, {v: v for v in values}, module=__name__)
    cls.__doc__ = doc
    return cls


ParamsGroupMethod = _enum("ParamsGroupMethod", ["mup"], "How parameters are partitioned into optimizer groups.")
GradientCheckpointingMethod = _enum("GradientCheckpointingMethod", ["block"], "Granularity of activation recomputation.")
LRDecaySchedule = _enum(
    "LRDecaySchedule", ["constant", "cosine", "exponential", "linear", "power"], "Shape of the decay phase."
)
DatasetSplit = _enum("DatasetSplit", ["train", "val", "test"], "Dataset split.")
Mode = _enum("Mode", ["training", "inference", "unsharding", "distillation"], "What the entry point is doing.")
TuningMethod = _enum("TuningMethod", ["pretraining", "full_finetuning", "distillation"], "Training objective family.")
LossMask = _enum("LossMask", ["output_only", "no_mask"], "Which tokens of an example contribute to the loss.")
KLDivergenceMethod = _enum("KLDivergenceMethod", ["forward", "backward"], "Direction of the distillation KL term.")
ExperimentsTrackerName = _enum("ExperimentsTrackerName", ["aim", "wandb"], "Experiment tracker backend.")

# Kernel names are kept for configuration compatibility; each selects the native sm_100a kernel of the same
# role (for instance `rmsnorm_cute` turns on the fused RMSNorm kernel, `scattermoe` the grouped expert GEMM).
Kernel = _enum(
    "Kernel",
    [
        "causal_conv1d",
        "continuous_count_cute",
        "cross_entropy_cute",
        "fused_linear_cross_entropy_cute",
        "gru_cute",
        "pack_sequence_cute",
        "rmsnorm_cute",
        "rmsnorm_memory_efficient_cute",
        "rnn_cute",
        "swiglu_packed_cute",
        "unpack_sequence_cute",
        "flash_attention_2",
        "flash_attention_3",
        "mamba2_ssm",
        "scattermoe",
        "ladder_residual_overlapped_layer",
        # additions of this engine
        "gemm_tcgen05",
        "stickbreaking_attention",
        "rope_fused",
        "fused_block",
        "adamw_fused",
    ],
    "Switchable kernels.",
)

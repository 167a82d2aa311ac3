"""Shared utilities (parity: lm_engine/utils/__init__.py:9-79)."""

from __future__ import annotations

import logging

import torch

from .hf_hub import download_repo
from .logger import log_metrics, log_rank_0, print_rank_0, print_ranks_all, set_logger, warn_rank_0
from .loss_dict import MetricsTrackingDict
from .miscellaneous import ceil_div, divide_if_divisible, round_up
from .mixed_precision import normalize_dtype_string, string_to_torch_dtype, torch_dtype_to_string
from .packages import (
    is_aim_available,
    is_causal_conv1d_available,
    is_colorlog_available,
    is_cute_kernels_available,
    is_flash_attention_2_available,
    is_flash_attention_3_available,
    is_mamba_2_ssm_available,
    is_native_kernels_available,
    is_stickbreaking_available,
    is_torchao_available,
    is_triton_available,
    is_wandb_available,
    is_zstandard_available,
    log_environment,
)
from .parallel import ProcessGroupManager, get_pipeline_stage_ids_on_current_rank, is_tracking_rank, run_rank_n
from .pydantic import BaseArgs
from .safetensors import SafeTensorsWeightsManager
from .step_tracker import StepTracker
from .timers import DeviceTimer, max_over_ranks
from .tracking import ExperimentsTracker, ProgressBar
from .wrapper import get_module_class_from_name
from .yaml import load_yaml


def init_distributed(
    tensor_parallel_world_size: int = 1,
    pipeline_parallel_world_size: int = 1,
    data_parallel_replication_world_size: int | None = None,
    data_parallel_sharding_world_size: int | None = None,
    zero_stage: int = 3,
    timeout_minutes: int | None = None,
    use_async_tensor_parallel: bool = False,
    expert_parallel_world_size: int = 1,
) -> None:
    """Create the process groups and log the resulting topology."""
    ProcessGroupManager(
        tensor_parallel_world_size=tensor_parallel_world_size,
        pipeline_parallel_world_size=pipeline_parallel_world_size,
        data_parallel_replication_world_size=data_parallel_replication_world_size,
        data_parallel_sharding_world_size=data_parallel_sharding_world_size,
        zero_stage=zero_stage,
        timeout_minutes=timeout_minutes,
        use_async_tensor_parallel=use_async_tensor_parallel,
        expert_parallel_world_size=expert_parallel_world_size,
    )
    log_rank_0(logging.INFO, f"device mesh: {ProcessGroupManager.get_mesh()}")
    log_rank_0(logging.INFO, f"total ranks = {ProcessGroupManager.get_world_size()}")
    log_rank_0(logging.INFO, f"tensor parallel size = {ProcessGroupManager.get_tensor_parallel_world_size()}")
    log_rank_0(logging.INFO, f"pipeline parallel size = {ProcessGroupManager.get_pipeline_parallel_world_size()}")
    log_rank_0(logging.INFO, f"data parallel size = {ProcessGroupManager.get_data_parallel_world_size()}")
    log_rank_0(logging.INFO, f"expert parallel size = {ProcessGroupManager.get_expert_parallel_world_size()}")


def setup_tf32(use_tf32: bool = True) -> None:
    torch.backends.cuda.matmul.allow_tf32 = use_tf32
    torch.backends.cudnn.allow_tf32 = use_tf32

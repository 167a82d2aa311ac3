"""Probes for optional dependencies. Each probe imports lazily and caches its answer."""

from __future__ import annotations

import importlib
import importlib.metadata
import logging
from functools import lru_cache


@lru_cache(maxsize=None)
def _can_import(name: str) -> bool:
    try:
        importlib.import_module(name)
        return True
    except Exception:
        return False


def is_apex_available() -> bool:
    return _can_import("apex")


def is_aim_available() -> bool:
    return _can_import("aim")


def is_wandb_available() -> bool:
    return _can_import("wandb")


def is_colorlog_available() -> bool:
    return _can_import("colorlog")


def is_triton_available() -> bool:
    return _can_import("triton")


def is_cute_kernels_available() -> bool:
    """The external `cute_kernels` package is never required: the kernels of the same roles are native here."""
    return _can_import("cute_kernels")


def is_native_kernels_available() -> bool:
    """True when the in-tree sm_100a extension is built and a CUDA device is present."""
    import torch

    from ..ops.build import is_extension_built

    return torch.cuda.is_available() and is_extension_built()


def is_flash_attention_2_available() -> bool:
    return _can_import("flash_attn")


def is_flash_attention_3_available() -> bool:
    return _can_import("flash_attn_interface")


def is_causal_conv1d_available() -> bool:
    return _can_import("causal_conv1d")


def is_mamba_2_ssm_available() -> bool:
    return _can_import("mamba_ssm")


def is_torchao_available() -> bool:
    return _can_import("torchao")


def is_stickbreaking_available() -> bool:
    return _can_import("stickbreaking_attention")


def is_zstandard_available() -> bool:
    return _can_import("zstandard")


def is_pyarrow_available() -> bool:
    return _can_import("pyarrow")


def log_environment() -> None:
    """Write the installed distributions to the log (rank 0 only)."""
    from .logger import log_rank_0

    rows = sorted({f"{d.metadata['Name']}=={d.version}" for d in importlib.metadata.distributions() if d.metadata["Name"]})
    log_rank_0(logging.INFO, "------------------------ packages ------------------------")
    for row in rows:
        log_rank_0(logging.INFO, row)
    log_rank_0(logging.INFO, "-------------------- end of packages ---------------------")

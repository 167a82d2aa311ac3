"""Names <-> torch dtypes ("fp32" / "fp16" / "bf16"; "fp8" computes in bf16 outside the scaled GEMMs)."""

from __future__ import annotations

import torch

_NAME_TO_DTYPE = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp8": torch.bfloat16}
_DTYPE_TO_NAME = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}


def normalize_dtype_string(dtype: str) -> str:
    key = str(dtype).lower().replace("torch.", "")
    aliases = {"float32": "fp32", "float": "fp32", "float16": "fp16", "half": "fp16", "bfloat16": "bf16"}
    key = aliases.get(key, key)
    if key not in _NAME_TO_DTYPE:
        raise ValueError(f"unexpected dtype '{dtype}'")
    return key


def string_to_torch_dtype(dtype: str | None) -> torch.dtype | None:
    if dtype is None:
        return None
    return _NAME_TO_DTYPE[normalize_dtype_string(dtype)]


def torch_dtype_to_string(dtype: torch.dtype) -> str:
    if dtype not in _DTYPE_TO_NAME:
        raise ValueError(f"unexpected dtype '{dtype}'")
    return _DTYPE_TO_NAME[dtype]

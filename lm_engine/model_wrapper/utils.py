"""Input broadcast inside a tensor parallel group (parity: lm_engine/model_wrapper/utils.py:10-22)."""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..utils import ProcessGroupManager


def broadcast_tensor_parallel_input(tokens: torch.Tensor | None, shape: tuple[int, ...], dtype=torch.long) -> torch.Tensor:
    """Rank 0 of the tensor parallel group holds the batch; everyone else receives a copy of it."""
    device = ProcessGroupManager.get_device()
    if ProcessGroupManager.is_tensor_parallel_first_rank():
        tokens = tokens.to(device)
    else:
        tokens = torch.empty(shape, dtype=dtype, device=device)
    dist.broadcast(tokens, src=ProcessGroupManager.get_tensor_parallel_first_rank(),
                   group=ProcessGroupManager.get_tensor_parallel_group())
    return tokens

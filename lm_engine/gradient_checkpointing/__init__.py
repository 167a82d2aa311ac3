"""Activation recomputation (parity: lm_engine/gradient_checkpointing/{__init__.py:17-23, block.py:17-41})."""

from __future__ import annotations

import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..enums import GradientCheckpointingMethod


class _CheckpointedBlock(nn.Module):
    def __init__(self, block: nn.Module, use_reentrant: bool) -> None:
        super().__init__()
        self.block = block
        self.use_reentrant = use_reentrant

    def forward(self, *args, **kwargs):
        if not self.training:
            return self.block(*args, **kwargs)
        return checkpoint(self.block, *args, use_reentrant=self.use_reentrant, **kwargs)


def block_checkpointing(model: nn.Module, block_name: str, num_blocks: int | None = None, use_reentrant: bool = False) -> None:
    """Recompute the first ``num_blocks`` (default: all) blocks of class ``block_name`` in backward. The wrapper
    keeps parameter names unchanged by replacing ``forward`` instead of inserting a module."""
    done = 0
    for module in model.modules():
        if type(module).__name__ != block_name:
            continue
        if num_blocks is not None and done >= num_blocks:
            break
        inner = module.forward

        def wrapped(*args, __inner=inner, __module=module, **kwargs):
            if not __module.training:
                return __inner(*args, **kwargs)
            return checkpoint(__inner, *args, use_reentrant=use_reentrant, **kwargs)

        module.forward = wrapped
        done += 1


_METHODS = {GradientCheckpointingMethod.block: block_checkpointing}


def apply_gradient_checkpointing(model: nn.Module, gradient_checkpointing_method: GradientCheckpointingMethod | None,
                                 **kwargs) -> None:
    if gradient_checkpointing_method is None:
        return
    _METHODS[gradient_checkpointing_method](model, **kwargs)

"""Parameter markers read by the optimizer param-group builder (parity: lm_engine/hf_models/parameter.py:8-30)."""

from __future__ import annotations

import torch.nn as nn

_NO_WEIGHT_DECAY = "_no_weight_decay"
_MUP_LR = "_has_mup_learning_rate"


def mark_parameter_as_no_weight_decay(parameter: nn.Parameter | None) -> nn.Parameter | None:
    if parameter is not None:
        setattr(parameter, _NO_WEIGHT_DECAY, True)
    return parameter


def mark_parameter_as_mup_learning_rate(parameter: nn.Parameter | None) -> nn.Parameter | None:
    if parameter is not None:
        setattr(parameter, _MUP_LR, True)
    return parameter


def is_parameter_with_no_weight_decay(parameter: nn.Parameter | None) -> bool:
    return getattr(parameter, _NO_WEIGHT_DECAY, False)


def is_parameter_with_mup_learning_rate(parameter: nn.Parameter | None) -> bool:
    return getattr(parameter, _MUP_LR, False)


def copy_markers(source, target) -> None:
    for name in (_NO_WEIGHT_DECAY, _MUP_LR):
        if getattr(source, name, False):
            setattr(target, name, True)

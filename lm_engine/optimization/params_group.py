"""Partition of parameters into optimizer groups (parity: lm_engine/optimization/params_group.py:16-135).

``normal`` uses the optimizer defaults, ``no_weight_decay`` (biases, norm weights: parameters carrying the
no-weight-decay marker) sets ``weight_decay = 0`` and, with ``params_group_method: mup``, parameters carrying the
muP marker form group ``mup`` with ``lr / m_width``. Names are sorted inside each group for determinism.
"""

from __future__ import annotations

import torch.nn as nn

from ..enums import ParamsGroupMethod
from ..hf_models.parameter import is_parameter_with_mup_learning_rate, is_parameter_with_no_weight_decay

GROUP_ORDER = ["normal", "no_weight_decay", "mup"]


def default_group_of(name: str, parameter: nn.Parameter) -> str:
    return "no_weight_decay" if is_parameter_with_no_weight_decay(parameter) else "normal"


def mup_group_of(name: str, parameter: nn.Parameter) -> str:
    if is_parameter_with_mup_learning_rate(parameter):
        return "mup"
    return default_group_of(name, parameter)


def get_group_function(params_group_method: ParamsGroupMethod | None):
    if params_group_method is None:
        return default_group_of
    if params_group_method == ParamsGroupMethod.mup:
        return mup_group_of
    raise ValueError(f"unexpected `params_group_method` {params_group_method}")


def group_overrides(group: str, optimizer_class_args: dict, m_width: float | None) -> dict:
    if group == "no_weight_decay":
        return {"weight_decay": 0}
    if group == "mup":
        if m_width is None:
            raise ValueError("the mup parameter group needs config.m_width (and init_method: mup)")
        return {"lr": optimizer_class_args["lr"] / m_width}
    return {}


def get_param_groups_with_names(model: nn.Module, params_group_method: ParamsGroupMethod | None) -> dict[str, list[str]]:
    """``{group name: sorted parameter names}`` - what the param-group golden files pin."""
    if params_group_method == ParamsGroupMethod.mup:
        config = getattr(model, "config", None)
        if config is not None and getattr(config, "init_method", "normal") != "mup":
            raise ValueError("both the model init method and the params group method must be mup")
    fn = get_group_function(params_group_method)
    names = {g: [] for g in (GROUP_ORDER if params_group_method == ParamsGroupMethod.mup else GROUP_ORDER[:2])}
    student = model.model if getattr(model, "has_teacher_model", lambda: False)() else model
    for name, parameter in student.named_parameters():
        names[fn(name, parameter)].append(name)
    return {g: sorted(v) for g, v in names.items()}


def get_torch_param_groups(model: nn.Module, optimizer_class_args: dict, params_group_method: ParamsGroupMethod | None) -> list[dict]:
    """Parameter groups over the module's own parameters (used when no sharded engine owns the model)."""
    by_name = get_param_groups_with_names(model, params_group_method)
    student = model.model if getattr(model, "has_teacher_model", lambda: False)() else model
    lookup = dict(student.named_parameters())
    m_width = getattr(getattr(model, "config", None), "m_width", None)
    groups = []
    for g, names in by_name.items():
        entry = {"params": [lookup[n] for n in names]}
        entry.update(group_overrides(g, optimizer_class_args, m_width))
        groups.append(entry)
    return groups

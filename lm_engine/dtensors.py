"""Conversions between plain tensors and DTensors (API parity: lm_engine/dtensors.py:12-86).

The training path of this engine does not use DTensors (layout crossings are explicit collectives); they appear at the
checkpoint boundary, where shards are described to ``torch.distributed.checkpoint``, and these helpers are kept for
code written against the reference.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor, Placement

from .utils import ProcessGroupManager


def _as_list(placement):
    return [placement] if isinstance(placement, Placement) else placement


def tensor_to_dtensor(tensor: torch.Tensor, device_mesh: DeviceMesh, current_placement, desired_placement=None,
                      run_check: bool = False) -> DTensor:
    if isinstance(tensor, DTensor):
        return tensor
    out = DTensor.from_local(tensor, device_mesh=device_mesh, run_check=run_check, placements=_as_list(current_placement))
    if desired_placement is not None:
        out = out.redistribute(device_mesh=device_mesh, placements=_as_list(desired_placement), async_op=True)
    return out


def dtensor_to_tensor(dtensor, device_mesh: DeviceMesh | None = None, desired_placement=None, grad_placement=None) -> torch.Tensor:
    if not isinstance(dtensor, DTensor):
        return dtensor
    if desired_placement is not None:
        assert device_mesh is not None
        dtensor = dtensor.redistribute(device_mesh=device_mesh, placements=_as_list(desired_placement), async_op=True)
    return dtensor.to_local(grad_placements=_as_list(grad_placement) if grad_placement is not None else None)


@torch.no_grad()
def modify_state_dict_to_dtensor_dict(module: nn.Module, state_dict: dict, prefix: str, strip_keys: bool) -> dict:
    """Wrap the plain tensors of ``state_dict`` like the (DTensor) parameters of ``module`` they are meant for."""
    own = module.state_dict()
    out = {}
    for key, tensor in state_dict.items():
        if not key.startswith(prefix):
            continue
        name = key[len(prefix):] if strip_keys and prefix else key
        param = own[name]
        if isinstance(tensor, DTensor) or not isinstance(param, DTensor):
            out[key] = tensor
        else:
            out[key] = tensor_to_dtensor(tensor, device_mesh=param.device_mesh, current_placement=param.placements)
    return out


def use_async_tensor_parallel() -> bool:
    return ProcessGroupManager.is_async_tensor_parallel_enabled()

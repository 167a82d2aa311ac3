"""Optimizer factory (parity: lm_engine/optimization/optimizer.py:26-97).

``class_name`` selects a ``torch.optim`` class by the reference's names. When a model is owned by the sharded
training engine the optimizer is built over the engine's flat fp32 segments (one tensor per unit and parameter
group), which makes every torch optimizer shard-aware for free; ``TorchAdamW`` / ``TorchAdam`` additionally get the
fused kernel (``FusedAdamW``): decay, moments, update, bf16 write-back and gradient clearing in one pass.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.optim import ASGD, LBFGS, SGD, Adadelta, Adagrad, Adam, Adamax, AdamW, NAdam, Optimizer, RAdam, RMSprop, Rprop

from .. import ops
from ..containers import BackwardHookOptimizerContainer, ModelContainer, OptimizerContainer
from ..enums import ParamsGroupMethod
from .params_group import GROUP_ORDER, get_torch_param_groups, group_overrides

_OPTIMIZER_CLASSES = {
    "TorchAdadelta": Adadelta, "TorchAdagrad": Adagrad, "TorchAdam": Adam, "TorchAdamax": Adamax, "TorchAdamW": AdamW,
    "TorchASGD": ASGD, "TorchLBFGS": LBFGS, "TorchNAdam": NAdam, "TorchRAdam": RAdam, "TorchRMSprop": RMSprop,
    "TorchRprop": Rprop, "TorchSGD": SGD,
}


class FusedAdamW(Optimizer):
    """AdamW over flat fp32 segments with this library's fused kernel.

    ``grad_scale`` (a one-element device tensor, typically the clipping coefficient) and ``grad_mul`` (a host float,
    typically 1 / data-parallel size) multiply the gradient inside the kernel, so clipping and averaging never touch
    memory. A segment may carry ``_lm_engine_segment.compute``: the bf16 copy refreshed in the same pass.
    """

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 decoupled: bool = True) -> None:
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.decoupled = decoupled
        self.grad_scale: torch.Tensor | None = None
        self.grad_mul: float = 1.0
        self.writes_compute_copy = True

    @torch.no_grad()
    def step(self, closure=None):
        loss = None if closure is None else closure()
        # True when every updated segment that has peers stored its result on all of them (see adamw_step_bcast)
        self.last_step_broadcast = True
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                state["step"] += 1
                seg = getattr(p, "_lm_engine_segment", None)
                target = None if seg is None else seg.compute
                bcast = None if seg is None else seg.broadcast
                if bcast is not None and p.is_cuda and ops.native_available() and p.numel() % 8 == 0 and self.decoupled:
                    # update + store of the bf16 result into every rank's compute copy (no parameter all-gather)
                    ops.native().adamw_step_bcast(p.data, state["exp_avg"], state["exp_avg_sq"], p.grad, bcast[0], bcast[1], bcast[2],
                                                  group["lr"], beta1, beta2, group["eps"], group["weight_decay"], state["step"],
                                                  self.grad_scale, self.grad_mul, True)
                elif p.is_cuda and ops.native_available() and p.numel() % 4 == 0 and self.decoupled:
                    self.last_step_broadcast = False
                    ops.native().adamw_step(p.data, state["exp_avg"], state["exp_avg_sq"], p.grad, target, group["lr"], beta1,
                                            beta2, group["eps"], group["weight_decay"], state["step"], self.grad_scale,
                                            self.grad_mul, True)
                elif not p.is_cuda and self.decoupled and hasattr(torch, "_fused_adamw_") and p.dtype == torch.float32:
                    # cpu_offload: the master shard, its moments and the staged gradient live on the host
                    self.last_step_broadcast = False
                    self._step_host(p, state, group, target)
                else:
                    self.last_step_broadcast = False
                    self._step_torch(p, state, group, target)
        return loss

    def _step_host(self, p, state, group, target) -> None:
        """One pass of PyTorch's fused CPU AdamW over a host-resident segment (instead of a dozen element-wise passes),
        then the copy of the result into the device's compute shard."""
        g = p.grad
        factor = self.grad_mul
        if self.grad_scale is not None:
            if getattr(self, "_host_scale_of", None) is not self.grad_scale or self._host_scale_step != state["step"]:
                # one device-to-host read of the clipping coefficient per optimizer step, not per segment
                self._host_scale, self._host_scale_of, self._host_scale_step = float(self.grad_scale), self.grad_scale, state["step"]
            factor = factor * self._host_scale
        if factor != 1.0:
            g.mul_(factor)
        beta1, beta2 = group["betas"]
        step = torch.tensor(float(state["step"]))
        torch._fused_adamw_([p], [g], [state["exp_avg"]], [state["exp_avg_sq"]], [], [step], lr=group["lr"], beta1=beta1, beta2=beta2,
                            weight_decay=group["weight_decay"], eps=group["eps"], amsgrad=False, maximize=False)
        if target is not None:
            target.copy_(p)
        g.zero_()

    def _step_torch(self, p, state, group, target) -> None:
        beta1, beta2 = group["betas"]
        g = p.grad * self.grad_mul
        if self.grad_scale is not None:
            g = g * self.grad_scale.to(g.device)
        step = state["step"]
        if self.decoupled:
            p.mul_(1 - group["lr"] * group["weight_decay"])
        elif group["weight_decay"] != 0:
            g = g + group["weight_decay"] * p
        state["exp_avg"].mul_(beta1).add_(g, alpha=1 - beta1)
        state["exp_avg_sq"].mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1 = 1 - beta1**step
        bc2 = 1 - beta2**step
        denom = (state["exp_avg_sq"].sqrt() / (bc2**0.5)).add_(group["eps"])
        p.addcdiv_(state["exp_avg"], denom, value=-group["lr"] / bc1)
        if target is not None:
            target.copy_(p)
        p.grad.zero_()


def _engine_param_groups(engine, optimizer_class_args: dict, m_width: float | None) -> list[dict]:
    """One optimizer group per parameter group that exists anywhere in the model - also on ranks whose shards hold no
    element of it, so that the group list (and with it scheduler / optimizer state) is the same on every rank and
    for every world size."""
    groups = []
    by_group = engine.segments_by_group()
    present = {slot.group for _, slot in engine.named_slots()}
    for name in GROUP_ORDER:
        if name not in present:
            continue
        entry = {"params": [seg.master for seg in by_group.get(name, [])], "name": name}
        entry.update(group_overrides(name, optimizer_class_args, m_width))
        groups.append(entry)
    return groups


def build_optimizer(model: nn.Module, optimizer_class_name: str, optimizer_class_args: dict,
                    params_group_method: ParamsGroupMethod | None) -> Optimizer:
    if optimizer_class_name not in _OPTIMIZER_CLASSES:
        raise ValueError(f"invalid class_name ({optimizer_class_name}) for optimizer")
    args = dict(optimizer_class_args)
    engine = getattr(model, "_lm_engine", None)
    m_width = getattr(getattr(model, "config", None), "m_width", None)
    if engine is None:
        groups = get_torch_param_groups(model, args, params_group_method)
        return _OPTIMIZER_CLASSES[optimizer_class_name](groups, **args)

    groups = _engine_param_groups(engine, args, m_width)
    if optimizer_class_name in ("TorchAdamW", "TorchAdam") and not args.get("amsgrad", False):
        fused_args = {k: v for k, v in args.items() if k in ("lr", "betas", "eps", "weight_decay")}
        if optimizer_class_name == "TorchAdam":
            fused_args.setdefault("weight_decay", 0.0)
        optimizer = FusedAdamW(groups, decoupled=optimizer_class_name == "TorchAdamW", **fused_args)
    else:
        optimizer = _OPTIMIZER_CLASSES[optimizer_class_name](groups, **args)
        optimizer.writes_compute_copy = False
    engine.optimizer = optimizer
    return optimizer


def get_optimizer_container(optimizer_class_name: str, optimizer_class_args: dict, model_container: ModelContainer,
                            params_group_method: ParamsGroupMethod | None = None,
                            use_optimizer_with_backward_hook: bool = False) -> OptimizerContainer:
    if use_optimizer_with_backward_hook:
        # experimental: every parameter owns an optimizer that is stepped as soon as its gradient is ready
        for model in model_container:
            for param in model.parameters():
                param._optimizer = _OPTIMIZER_CLASSES[optimizer_class_name]([param], **optimizer_class_args)

                def _step(p: nn.Parameter) -> None:
                    p._optimizer.step()
                    p._optimizer.zero_grad()

                param.register_post_accumulate_grad_hook(_step)
        return BackwardHookOptimizerContainer([None] * len(model_container))
    return OptimizerContainer(
        [build_optimizer(model, optimizer_class_name, optimizer_class_args, params_group_method) for model in model_container]
    )

"""Learning-rate schedules: warmup -> constant -> decay -> floor, as multiplicative factors for ``LambdaLR``.

Parity: lm_engine/optimization/scheduler.py:31-252. Shapes of the decay phase (x = steps into the phase, t = its
length, f = ``lr_decay_factor``):

* cosine      ``(1 - f) * (1 + cos(pi x / t)) / 2 + f``
* linear      ``1 + (f - 1) x / t``
* exponential ``a e^(-x/t) + b`` with a, b chosen so that the factor is 1 at x = 0 and f at x = t (it keeps decaying)
* power (arXiv 2408.13359) ``min(1, (a / lr) (c * steps)^b)`` over the absolute step count, with a linear warmup to
  the value the power law takes at the end of warmup.
"""

from __future__ import annotations

import math

from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR

from ..containers import BackwardHookOptimizerContainer, LRSchedulerContainer
from ..enums import LRDecaySchedule


class PhasedSchedule:
    """Pure function ``step -> factor``; separate from LambdaLR so that it can be evaluated and tested directly."""

    def __init__(self, style: LRDecaySchedule, num_warmup_steps: int, num_constant_steps: int, num_decay_steps: int | None,
                 num_training_steps: int, lr_decay_factor: float, base_lr: float | None = None, a: float | None = None,
                 b: float | None = None, c: float | None = None) -> None:
        self.style = style
        self.warmup_end = num_warmup_steps
        self.constant_end = num_warmup_steps + num_constant_steps
        self.decay_end = num_training_steps if num_decay_steps is None else self.constant_end + num_decay_steps
        self.floor = lr_decay_factor
        if style == LRDecaySchedule.constant and num_decay_steps not in (0,):
            raise ValueError("num_decay_steps should be 0 for the constant schedule")
        if style == LRDecaySchedule.power:
            if num_constant_steps != 0:
                raise ValueError("num_constant_steps should be 0 for the power schedule")
            if None in (a, b, c, base_lr):
                raise ValueError("the power schedule needs extra_lr_scheduler_args a, b and c")
            self.a_over_lr, self.b, self.c = a / base_lr, b, c
            self.warmup_peak = min(1.0, self._power(num_warmup_steps)) if num_warmup_steps > 0 else 1.0

    def _power(self, steps: int) -> float:
        return self.a_over_lr * (steps * self.c) ** self.b

    def __call__(self, step: int) -> float:
        in_warmup = self.warmup_end > 0 and step <= self.warmup_end
        if self.style == LRDecaySchedule.power:
            if in_warmup:
                return self.warmup_peak * step / self.warmup_end
            return min(1.0, self._power(step))
        if in_warmup:
            return step / self.warmup_end
        if self.style == LRDecaySchedule.constant or step <= self.constant_end:
            return 1.0
        x = step - self.constant_end
        t = self.decay_end - self.constant_end
        f = self.floor
        if self.style == LRDecaySchedule.exponential:
            a = (1 - f) * math.e / (math.e - 1)
            b = (f * math.e - 1) / (math.e - 1)
            return a * math.exp(-x / t) + b
        if step > self.decay_end:
            return f
        if self.style == LRDecaySchedule.cosine:
            return (1 - f) * (1 + math.cos(math.pi * x / t)) / 2 + f
        if self.style == LRDecaySchedule.linear:
            return 1 + (f - 1) * x / t
        raise ValueError(f"invalid lr_decay_style ({self.style})")


def build_lr_scheduler(optimizer: Optimizer, num_warmup_steps: int, num_constant_steps: int, num_decay_steps: int | None,
                       num_training_steps: int, lr_decay_style: LRDecaySchedule, lr_decay_factor: float,
                       extra_lr_scheduler_args: dict | None = None, last_epoch: int = -1) -> LambdaLR:
    schedule = PhasedSchedule(lr_decay_style, num_warmup_steps, num_constant_steps, num_decay_steps, num_training_steps,
                              lr_decay_factor, base_lr=optimizer.param_groups[0]["lr"], **(extra_lr_scheduler_args or {}))
    return LambdaLR(optimizer, lr_lambda=schedule, last_epoch=last_epoch)


def get_scheduler_container(model_container, optimizer_container, num_warmup_steps: int, num_constant_steps: int,
                            num_decay_steps: int | None, num_training_steps: int, lr_decay_style: LRDecaySchedule,
                            lr_decay_factor: float, extra_lr_scheduler_args: dict, use_optimizer_with_backward_hook: bool = False,
                            last_epoch: int = -1):
    if lr_decay_style not in list(LRDecaySchedule):
        raise ValueError(f"invalid lr_decay_style ({lr_decay_style})")
    kwargs = dict(num_warmup_steps=num_warmup_steps, num_constant_steps=num_constant_steps, num_decay_steps=num_decay_steps,
                  num_training_steps=num_training_steps, lr_decay_style=lr_decay_style, lr_decay_factor=lr_decay_factor,
                  extra_lr_scheduler_args=extra_lr_scheduler_args, last_epoch=last_epoch)
    if use_optimizer_with_backward_hook:
        for model in model_container:
            for param in model.parameters():
                param._lr_scheduler = build_lr_scheduler(param._optimizer, **kwargs)
                param.register_post_accumulate_grad_hook(lambda p: p._lr_scheduler.step())
        return BackwardHookOptimizerContainer([None] * len(model_container))
    return LRSchedulerContainer([build_lr_scheduler(optimizer, **kwargs) for optimizer in optimizer_container])

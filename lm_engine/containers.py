"""List containers with one entry per local pipeline stage (parity: lm_engine/containers.py:12-77)."""

from __future__ import annotations

import logging

import torch.nn as nn


class _Container:
    def __init__(self, items: list) -> None:
        self.items = list(items)

    def __iter__(self):
        return iter(self.items)

    def __getitem__(self, index: int):
        return self.items[index]

    def __setitem__(self, index: int, value) -> None:
        self.items[index] = value

    def __len__(self) -> int:
        return len(self.items)

    def __repr__(self) -> str:
        body = ", ".join(repr(i) for i in self.items)
        return f"{type(self).__name__}([{body}])"


class ModelContainer(_Container):
    def train(self) -> "ModelContainer":
        for model in self:
            model.train()
        return self

    def eval(self) -> "ModelContainer":
        for model in self:
            model.eval()
        return self


class OptimizerContainer(_Container):
    def step(self) -> None:
        for optimizer in self:
            optimizer.step()

    def zero_grad(self) -> None:
        for optimizer in self:
            optimizer.zero_grad()


class LRSchedulerContainer(_Container):
    def step(self) -> None:
        for scheduler in self:
            scheduler.step()


class BackwardHookOptimizerContainer(_Container):
    """Stand-in used when each parameter carries its own optimizer stepped from a gradient hook."""

    def step(self) -> None:
        return None

    def zero_grad(self) -> None:
        return None

    def state_dict(self):
        return {}


def log_model_optimizer_container(model_container: ModelContainer, optimizer_container: OptimizerContainer) -> None:
    from .utils import log_rank_0

    log_rank_0(logging.INFO, "model container:")
    for model in model_container:
        log_rank_0(logging.INFO, str(model))
    log_rank_0(logging.INFO, "optimizer container:")
    for optimizer in optimizer_container:
        log_rank_0(logging.INFO, str(optimizer))

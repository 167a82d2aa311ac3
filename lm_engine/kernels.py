"""Kernel switchboard (parity: lm_engine/kernels.py:21-76).

``enable_kernels([...])`` is a context manager that swaps the active set, ``enable_all_kernels()`` turns on every
kernel except the ladder-residual overlap, and ``is_kernel_allowed(k)`` is what layers consult. Setting the
environment variable ``ENABLE_ALL_CUTE_KERNELS`` enables everything from process start.
"""

from __future__ import annotations

import os
from contextlib import contextmanager

import torch

from .enums import Kernel

_ALL_BUT_LADDER = {k for k in Kernel if k != Kernel.ladder_residual_overlapped_layer}


def _truthy(value: str | None) -> bool:
    return value is not None and value.strip().lower() in ("1", "true", "yes", "on")


_ACTIVE: set[Kernel] = set(_ALL_BUT_LADDER) if _truthy(os.environ.get("ENABLE_ALL_CUTE_KERNELS")) else set()


def is_kernel_allowed(kernel: Kernel) -> bool:
    return kernel in _ACTIVE


def get_enabled_kernels() -> set[Kernel]:
    return set(_ACTIVE)


@contextmanager
def enable_kernels(kernels: list[Kernel] | set[Kernel]):
    global _ACTIVE
    previous = _ACTIVE
    _ACTIVE = {Kernel(k) if not isinstance(k, Kernel) else k for k in kernels}
    try:
        yield
    finally:
        _ACTIVE = previous


@contextmanager
def enable_all_kernels():
    with enable_kernels(_ALL_BUT_LADDER):
        yield


class _BackwardWait(torch.autograd.Function):
    """Identity whose backward materialises an in-flight collective result before handing it on."""

    @staticmethod
    def forward(ctx, x: torch.Tensor) -> torch.Tensor:
        return x

    @staticmethod
    def backward(ctx, grad: torch.Tensor) -> torch.Tensor:
        return _materialize(grad)


def _materialize(x: torch.Tensor) -> torch.Tensor:
    try:
        from torch.distributed._functional_collectives import AsyncCollectiveTensor
    except Exception:  # pragma: no cover
        return x
    if isinstance(x, AsyncCollectiveTensor):
        return x.wait()
    return x


def wait_for_ACT(x: torch.Tensor, wait_in_forward: bool, wait_in_backward: bool) -> torch.Tensor:
    """Make sure an asynchronous collective result is complete before a non-torch kernel reads it."""
    if wait_in_forward:
        x = _materialize(x)
    if wait_in_backward and x.requires_grad:
        x = _BackwardWait.apply(x)
    return x

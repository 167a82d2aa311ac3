"""Per-site device timing and NVTX ranges for the explicit kernel schedules.

``with site("c_fc+swiglu"):`` around a launch site does nothing unless switched on:

* ``enable_timing()`` brackets every site with CUDA events on the current stream; ``report()`` returns, per site, the
  number of visits and the summed device time. That is how the per-kernel time budget of a training step is taken
  under the real clocks and cache state of the step (no profiler, no serialisation).
* ``enable_nvtx()`` (or ``LM_ENGINE_NVTX=1`` in the environment) pushes an NVTX range per site, so that a timeline
  tool shows the schedule with names instead of anonymous kernels.

Both are process-wide switches read at every site, so they can be flipped between steps.
"""

from __future__ import annotations

import os
from collections import defaultdict

import torch

_TIMING = False
_NVTX = os.environ.get("LM_ENGINE_NVTX", "0") == "1"
_EVENTS: dict[str, list[tuple[torch.cuda.Event, torch.cuda.Event]]] = defaultdict(list)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _Null()


class _Site:
    __slots__ = ("name", "start")

    def __init__(self, name: str) -> None:
        self.name = name
        self.start = None

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)
        if _TIMING:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _EVENTS[self.name].append((self.start, end))
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        return False


def site(name: str):
    """Context manager around one launch site (free when timing and NVTX are off)."""
    if not (_TIMING or _NVTX):
        return _NULL
    return _Site(name)


def enable_timing(on: bool = True) -> None:
    global _TIMING
    _TIMING = on and torch.cuda.is_available()
    if on:
        _EVENTS.clear()


def enable_nvtx(on: bool = True) -> None:
    global _NVTX
    _NVTX = on and torch.cuda.is_available()


def report() -> dict[str, dict[str, float]]:
    """``{site: {"calls": n, "ms": summed device time}}`` of everything recorded since ``enable_timing()``; synchronises."""
    torch.cuda.synchronize()
    out = {}
    for name, pairs in _EVENTS.items():
        out[name] = {"calls": len(pairs), "ms": sum(a.elapsed_time(b) for a, b in pairs)}
    return out

"""Device-side step timing: CUDA events on the launching stream, max over ranks."""

from __future__ import annotations

import time

import torch
import torch.distributed as dist


class DeviceTimer:
    """Brackets a region with CUDA events (falls back to the host clock on CPU)."""

    def __init__(self, device: torch.device | None = None) -> None:
        self.use_cuda = torch.cuda.is_available() and (device is None or device.type == "cuda")
        self._start = None
        self._end = None
        self._t0 = 0.0
        self._elapsed = 0.0

    def start(self) -> None:
        if self.use_cuda:
            self._start = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self.use_cuda:
            self._end.record()
        else:
            self._elapsed = time.perf_counter() - self._t0

    def elapsed_ms(self) -> float:
        if self.use_cuda:
            self._end.synchronize()
            return self._start.elapsed_time(self._end)
        return self._elapsed * 1e3


def max_over_ranks(value: float, group=None) -> float:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return value
    device = "cuda" if dist.get_backend(group) == "nccl" or "nccl" in str(dist.get_backend(group)) else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.item()

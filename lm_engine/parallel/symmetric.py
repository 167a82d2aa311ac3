"""Peer memory over NVLink: symmetric buffers, a bounded device-side barrier and the collectives built on them.

A :class:`PeerGroup` belongs to one process group. Buffers come from torch's symmetric-memory allocator (same layout on
every rank, every peer's copy mapped into this process; bound to an NVSwitch multicast object when the fabric supports
it), so kernels get one address per rank and optionally one multicast address. The kernels are in ``csrc/comm/peer.cu``:

``barrier``            epoch flags with release/acquire at system scope; the wait is bounded by wall time and reports
                       a status code (``check()`` raises on the host) instead of hanging when a rank is missing.
``reduce_scatter_f32`` sum of every rank's copy of one region: ``multimem.ld_reduce`` (summed in the switch) or plain
                       16-byte peer loads summed in rank order.
``adamw_step_bcast``   the optimizer update of this rank's fp32 shard whose bf16 result is stored into every rank's
                       compute copy (``multimem.st`` or one peer store per rank): the parameter all-gather costs no
                       separate pass.
``all_gather``         pull of the other ranks' shards, for optimizers that do not write the compute copy themselves.

``LM_ENGINE_PEER_MULTIMEM=0`` forces the plain peer path; ``LM_ENGINE_PEER_TIMEOUT_SECONDS`` sets the barrier limit.
Multi-rank tests that let a rank leave use the plain path and no multicast binding
(``TORCH_SYMM_MEM_DISABLE_MULTICAST=1``).
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import ops
from ..utils import log_rank_0

_CONTROL_WORDS = 64  # >= kMaxPeers flag words, padded to 256 bytes
_GROUPS: dict[int, "PeerGroup"] = {}


@dataclass
class PeerBuffer:
    """A tensor of this rank plus the addresses of the same allocation on every rank of the group."""

    tensor: torch.Tensor
    ptrs: list[int]
    multicast_ptr: int
    owner: "PeerGroup" = field(repr=False, default=None)
    handle: object = field(repr=False, default=None)

    def ptrs_at(self, byte_offset: int) -> list[int]:
        return [p + byte_offset for p in self.ptrs]

    def multicast_at(self, byte_offset: int) -> int:
        return self.multicast_ptr + byte_offset if self.multicast_ptr else 0

    def offset_of(self, view: torch.Tensor) -> int:
        """Byte offset of a view into this buffer."""
        offset = view.data_ptr() - self.tensor.data_ptr()
        assert 0 <= offset <= self.tensor.numel() * self.tensor.element_size()
        return offset


class PeerGroup:
    def __init__(self, group: dist.ProcessGroup | None, device: torch.device) -> None:
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = device
        self.use_multimem = os.environ.get("LM_ENGINE_PEER_MULTIMEM", "1") != "0"
        self.timeout_seconds = float(os.environ.get("LM_ENGINE_PEER_TIMEOUT_SECONDS", "60"))
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.control = self.alloc(_CONTROL_WORDS, torch.int32, zero=True)
        # a second set of flags with its own epoch counter: barriers issued on a side stream (collectives that run under
        # compute) must not interleave their epochs with those of the main stream
        self.side_epoch = 0
        self.side_control = self.alloc(_CONTROL_WORDS, torch.int32, zero=True)
        # the flags must read zero everywhere before the first barrier kernel publishes an epoch
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------------------------------------------------------
    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = True) -> PeerBuffer:
        import torch.distributed._symmetric_memory as symm

        try:
            symm.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        tensor = symm.empty(numel, dtype=dtype, device=self.device)
        if zero:
            tensor.zero_()
        handle = symm.rendezvous(tensor, self.group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        assert ptrs[self.rank] == tensor.data_ptr(), "symmetric buffer: local address is not the table's entry of this rank"
        multicast = int(getattr(handle, "multicast_ptr", 0) or 0) if self.use_multimem else 0
        return PeerBuffer(tensor, ptrs, multicast, self, handle)

    def barrier(self) -> None:
        """All ranks of the group have reached this point of their streams (and their earlier writes are visible)."""
        self.epoch += 1
        ops.native().peer_barrier(self.control.ptrs, self.rank, self.epoch & 0x7FFFFFFF, self.timeout_seconds, self.status)

    def side_barrier(self) -> None:
        """Same as :meth:`barrier` on the second set of flags; every rank must issue these from one (side) stream and in
        the same order."""
        self.side_epoch += 1
        ops.native().peer_barrier(self.side_control.ptrs, self.rank, self.side_epoch & 0x7FFFFFFF, self.timeout_seconds, self.status)

    def check(self) -> None:
        """Host-side check of the status word (synchronises with the device)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer barrier gave up after {self.timeout_seconds} s (status {code}): a rank of the group did not arrive")

    # ------------------------------------------------------------------------------------------------------------------
    def reduce_scatter_f32(self, buf: PeerBuffer, region: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
        """``out = scale * sum_r region_r`` where ``region`` is a view into ``buf`` (the same view on every rank)."""
        assert region.dtype == torch.float32 and out.dtype == torch.float32 and out.numel() == region.numel()
        offset = buf.offset_of(region)
        ops.native().peer_reduce_scatter_f32(buf.ptrs, buf.multicast_ptr, out, offset // 4, scale)

    def all_gather(self, buf: PeerBuffer, region: torch.Tensor, shard_numel: int) -> None:
        """``region`` (a view into ``buf`` of ``world * shard_numel`` elements) holds this rank's shard at its place;
        afterwards it holds everyone's."""
        offset = buf.offset_of(region)
        assert region.numel() == shard_numel * self.world
        ops.native().peer_all_gather(buf.ptrs_at(offset), self.rank, shard_numel * region.element_size(), region)


def get_peer_group(group: dist.ProcessGroup | None, device: torch.device) -> PeerGroup | None:
    """The peer group of a process group, created on first use; ``None`` when peer memory cannot be set up (the
    caller then stays on NCCL)."""
    if device.type != "cuda" or not ops.native_available() or not dist.is_initialized():
        return None
    key = id(group if group is not None else dist.group.WORLD)
    if key not in _GROUPS:
        try:
            _GROUPS[key] = PeerGroup(group, device)
        except Exception as error:  # allocator or fabric without peer access
            log_rank_0(logging.WARNING, f"peer memory is unavailable ({type(error).__name__}: {error}); collectives stay on NCCL")
            _GROUPS[key] = None
    return _GROUPS[key]


def check_all_peer_groups() -> None:
    """Raise if any peer group of this process recorded a barrier that gave up (synchronises with the device)."""
    for group in _GROUPS.values():
        if group is not None:
            group.check()

"""Peer-memory collectives: this engine's own kernels over NVLink instead of NCCL.

Buffers that take part are allocated from torch's symmetric-memory allocator (identical layout on every rank, every
peer's copy mapped into this process) and registered here. The kernels read peer shards with plain 16-byte loads
(never a TMA multicast load, never ``multimem`` on the reduce path used by fault-tolerance tests). Until a buffer is
registered the functions return False and the caller falls back to NCCL.
"""

from __future__ import annotations

import torch

_REGISTRY: dict[int, object] = {}


def register_symmetric(buf: torch.Tensor, handle) -> None:
    _REGISTRY[buf.data_ptr()] = handle


def lookup(buf: torch.Tensor):
    return _REGISTRY.get(buf.data_ptr())


def fused_reduce_scatter_in_place(buf: torch.Tensor, shard_numel: int, rank: int, group) -> bool:
    handle = lookup(buf)
    if handle is None:
        return False
    from .peer_kernels import peer_reduce_scatter

    return peer_reduce_scatter(buf, handle, shard_numel, rank)


def fused_all_gather_in_place(buf: torch.Tensor, shard_numel: int, rank: int, group) -> bool:
    handle = lookup(buf)
    if handle is None:
        return False
    from .peer_kernels import peer_all_gather

    return peer_all_gather(buf, handle, shard_numel, rank)

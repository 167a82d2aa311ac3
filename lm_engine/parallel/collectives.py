"""Collective shims shared by the CPU (gloo) and GPU (NCCL) paths; the peer-memory kernels that replace them on
NVLink are driven by the training engine directly (:mod:`lm_engine.parallel.symmetric`).

Every function works in place on one flat buffer split into ``world`` equal shards, which is how the sharded
training engine stores parameters and gradients. gloo lacks ``reduce_scatter_tensor`` and ``ReduceOp.AVG``, so
the CPU path all-reduces and lets every rank keep its slice; the results are identical.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _is_gloo(group) -> bool:
    backend = dist.get_backend(group)
    return "nccl" not in str(backend) and "gloo" in str(backend) or str(backend) == "gloo"


def _on_cpu(t: torch.Tensor) -> bool:
    return t.device.type == "cpu"


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    if group is not None and dist.get_world_size(group) == 1:
        return t
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def reduce_scatter_in_place(buf: torch.Tensor, shard_numel: int, rank: int, group=None, fused: bool = False) -> torch.Tensor:  # noqa: ARG001
    """Afterwards ``buf[rank * shard_numel : (rank + 1) * shard_numel]`` holds the sum over ranks of that slice."""
    shard = buf[rank * shard_numel : (rank + 1) * shard_numel]
    if _on_cpu(buf):
        dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
        return shard
    dist.reduce_scatter_tensor(shard, buf, op=dist.ReduceOp.SUM, group=group)
    return shard


def all_gather_in_place(buf: torch.Tensor, shard_numel: int, rank: int, group=None, fused: bool = False) -> torch.Tensor:
    """Every rank contributes ``buf[rank * shard_numel : (rank + 1) * shard_numel]``; afterwards ``buf`` is complete."""
    world = dist.get_world_size(group)
    shard = buf[rank * shard_numel : (rank + 1) * shard_numel]
    if _on_cpu(buf):
        pieces = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(pieces, shard.contiguous(), group=group)
        for r, piece in enumerate(pieces):
            if r != rank:
                buf[r * shard_numel : (r + 1) * shard_numel].copy_(piece)
        return buf
    dist.all_gather_into_tensor(buf, shard, group=group)
    return buf


def all_reduce_mean_scalars(values: torch.Tensor, group=None) -> torch.Tensor:
    """Average a small vector over a group (sum then divide: works on gloo too)."""
    world = 1 if group is None and not dist.is_initialized() else dist.get_world_size(group)
    if world > 1:
        dist.all_reduce(values, op=dist.ReduceOp.SUM, group=group)
        values = values / world
    return values

"""Dataloaders with resumable state and node-local dispatch (parity: lm_engine/data/dataloader.py:16-125)."""

from __future__ import annotations

from typing import Callable, Iterable

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Dataset, Sampler

from ..communication import Communication
from ..utils import ProcessGroupManager


class ResumableDataLoader(DataLoader):
    def state_dict(self) -> dict:
        state = {}
        if hasattr(self.dataset, "state_dict"):
            state["dataset"] = self.dataset.state_dict()
        if hasattr(self.sampler, "state_dict"):
            state["sampler"] = self.sampler.state_dict()
        return state

    def load_state_dict(self, state_dict: dict) -> None:
        if "dataset" in state_dict and hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(state_dict["dataset"])
        if "sampler" in state_dict and hasattr(self.sampler, "load_state_dict"):
            self.sampler.load_state_dict(state_dict["sampler"])


class DispatchingDataLoader(ResumableDataLoader):
    """One rank per node reads ``micro_batch x ranks_per_node`` samples and broadcasts them inside the node; every rank
    keeps its own slice. Only the source rank touches the dataset (and storage)."""

    def __init__(self, dataset: Dataset, batch_size: int | None = 1, sampler: Sampler | None = None,
                 batch_sampler: Sampler | None = None, num_workers: int = 0, collate_fn: Callable | None = None,
                 pin_memory: bool = False, drop_last: bool = False, source_broadcast_mapping: dict | None = None,
                 broadcast_world_size: int | None = None, static_shape_per_rank: tuple[int, ...] | None = None,
                 keys: list[str] = ("text",)) -> None:
        self.broadcast_world_size = broadcast_world_size
        self.all_source_ranks_and_broadcast_groups = source_broadcast_mapping or {}
        self.source_rank, self.broadcast_group = self._locate()
        self.is_source = ProcessGroupManager.get_global_rank() == self.source_rank
        self.local_rank_in_broadcast_group = ProcessGroupManager.get_global_rank() % max(broadcast_world_size or 1, 1)
        self.static_shape_per_rank = static_shape_per_rank
        self.keys = list(keys)
        self._micro = batch_size
        if self.is_source:
            full = None if batch_size is None else batch_size * (broadcast_world_size or 1)
            super().__init__(dataset, batch_size=full if batch_sampler is None else 1, sampler=sampler,
                             batch_sampler=batch_sampler, num_workers=num_workers, collate_fn=collate_fn,
                             pin_memory=pin_memory, drop_last=drop_last)
        else:
            self.dataset, self.sampler, self.batch_sampler = dataset, sampler, batch_sampler

    def _locate(self):
        me = ProcessGroupManager.get_global_rank()
        for source, group in self.all_source_ranks_and_broadcast_groups.items():
            if me in dist.get_process_group_ranks(group):
                return source, group
        return me, None

    def __iter__(self) -> Iterable:
        device = ProcessGroupManager.get_device()
        if self.is_source:
            for batch in super().__iter__():
                length = torch.tensor([1], device=device)
                dist.broadcast(length, src=self.source_rank, group=self.broadcast_group)
                out = {}
                for key in self.keys:
                    full = batch[key].to(device)
                    if self.static_shape_per_rank is None:
                        Communication.broadcast_object(tuple(full.shape), src=self.source_rank, group=self.broadcast_group)
                    dist.broadcast(full, src=self.source_rank, group=self.broadcast_group)
                    out[key] = full.chunk(self.broadcast_world_size)[self.local_rank_in_broadcast_group]
                yield out
            end = torch.tensor([0], device=device)
            dist.broadcast(end, src=self.source_rank, group=self.broadcast_group)
        else:
            while True:
                flag = torch.tensor([0], device=device)
                dist.broadcast(flag, src=self.source_rank, group=self.broadcast_group)
                if flag.item() == 0:
                    return
                out = {}
                for key in self.keys:
                    if self.static_shape_per_rank is None:
                        shape = Communication.broadcast_object(None, src=self.source_rank, group=self.broadcast_group)
                    else:
                        shape = (self.static_shape_per_rank[0] * self.broadcast_world_size, *self.static_shape_per_rank[1:])
                    full = torch.empty(shape, dtype=torch.long, device=device)
                    dist.broadcast(full, src=self.source_rank, group=self.broadcast_group)
                    out[key] = full.chunk(self.broadcast_world_size)[self.local_rank_in_broadcast_group]
                yield out

"""Resumable distributed sampler over a blend of datasets (parity: lm_engine/data/sampler.py:16-147).

Each epoch draws ``num_samples_by_dataset[i]`` indices from dataset ``i`` (proportional to ``data_sampling_ratio``;
whole passes plus a shuffled remainder when over-sampling), shuffles the union with a seed derived from
``seed + epoch``, pads or trims to a multiple of the replica count and strides by rank. ``state_dict`` records
epoch / position so that iteration can be resumed by replaying to the saved index.
"""

from __future__ import annotations

import math
from typing import Iterator

import torch
from torch.utils.data import DistributedSampler

from ..enums import DatasetSplit
from .base import BlendedDatasets


def _split_by_ratio(ratios: list[int], total: int) -> list[int]:
    r = torch.tensor(ratios, dtype=torch.float64)
    counts = (r / r.sum() * total).to(torch.long)
    counts[-1] = total - counts[:-1].sum()
    return counts.tolist()


class BlendedDistributedSampler(DistributedSampler):
    def __init__(self, dataset: BlendedDatasets, data_sampling_ratios: list[int], num_replicas: int, rank: int,
                 ignore_sampling_proportion_for_validation: bool = True, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False) -> None:
        super().__init__(dataset, num_replicas, rank, shuffle, seed, drop_last)
        self.sizes = dataset.get_num_examples_in_each_dataset()
        self.num_datasets = dataset.get_num_datasets()
        if dataset.split == DatasetSplit.val and ignore_sampling_proportion_for_validation:
            self.num_samples_by_dataset = list(self.sizes)
        else:
            self.num_samples_by_dataset = _split_by_ratio(data_sampling_ratios, len(dataset))
        self.generator = torch.Generator().manual_seed(seed) if shuffle else None
        self.starts = [sum(self.sizes[:i]) for i in range(self.num_datasets)]
        self.index = 0

    def _draw(self, wanted: int, size: int) -> torch.Tensor:
        if self.shuffle:
            self.generator.manual_seed(self.seed + self.epoch)
        if wanted < size:
            return torch.randperm(size, generator=self.generator)[:wanted] if self.shuffle else torch.arange(wanted)
        passes, rest = divmod(wanted, size)
        picks = torch.arange(size).repeat(passes)
        if rest > 0:
            extra = torch.randperm(size, generator=self.generator)[:rest] if self.shuffle else torch.arange(rest)
            picks = torch.cat([picks, extra])
        return picks

    def __iter__(self) -> Iterator[int]:
        indices: list[int] = []
        for d in range(self.num_datasets):
            indices.extend((self._draw(self.num_samples_by_dataset[d], self.sizes[d]) + self.starts[d]).tolist())
        if self.shuffle:
            self.generator.manual_seed(self.seed + self.epoch)
            order = torch.randperm(len(indices), generator=self.generator)
            indices = torch.tensor(indices)[order].tolist()
        if self.drop_last:
            indices = indices[: self.total_size]
        else:
            missing = self.total_size - len(indices)
            if missing > 0:
                indices += (indices * math.ceil(missing / len(indices)))[:missing]
        assert len(indices) == self.total_size
        mine = indices[self.rank : self.total_size : self.num_replicas]
        assert len(mine) == self.num_samples
        self.index = 0
        for i in mine:
            self.index += 1
            yield i
        self.set_epoch(self.epoch + 1)

    def state_dict(self) -> dict:
        state = {"epoch": self.epoch, "index": self.index}
        if self.shuffle:
            state["generator"] = self.generator.get_state()
        return state

    def load_state_dict(self, state_dict: dict) -> None:
        self.set_epoch(state_dict["epoch"])
        if self.shuffle:
            self.generator.set_state(state_dict["generator"])
        if state_dict["index"] == 0:
            return
        for _ in self:
            if self.index == state_dict["index"]:
                break

    def __repr__(self) -> str:
        lines = []
        for i, dataset in enumerate(self.dataset.datasets):
            n = self.num_samples_by_dataset[i]
            lines.append(f"samples of {type(dataset).__name__} ({dataset.data_name}) per epoch of the mixture = {n} "
                         f"({n / max(len(dataset), 1):.3f} epochs of that dataset)")
        return "\n".join(lines)

"""Blending of several token stores by weight, the dataset configs and the builder that is aware of ranks.

Parity: lm_engine/data/megatron/blended_dataset.py:21-166, blended_megatron_dataset_config.py:12-115,
blended_megatron_dataset_builder.py:23-435.
"""

from __future__ import annotations

import hashlib
import json
import logging
import math
import os
import re
from collections import OrderedDict
from copy import deepcopy
from dataclasses import dataclass, field

import numpy as np
import torch

from ...utils import ProcessGroupManager, log_rank_0
from .indexed_dataset import MMapIndexedDataset
from .utils import Split, build_blending_indices, normalize


# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class BlendedMegatronDatasetConfig:
    """``blend``: one prefix or a flat ``[weight, prefix, weight, prefix, ...]`` list used with ``split``
    (``"98,1,1"``-style weights of train/valid/test); ``blend_per_split``: one such list per split instead."""

    is_built_on_rank: bool
    random_seed: int
    sequence_length: int
    name: str | None = None
    blend: list[str] | None = None
    blend_per_split: list[list[str] | None] | None = None
    split: str | None = None
    split_vector: list[float] | None = field(init=False, default=None)
    path_to_cache: str | None = None
    node_uses_local_storage: bool = False

    def __post_init__(self) -> None:
        if ProcessGroupManager.get_global_rank() == 0:
            assert self.is_built_on_rank, "is_built_on_rank must be True when global rank = 0"
        if self.blend_per_split is not None and any(self.blend_per_split):
            assert self.blend is None, "blend and blend_per_split are incompatible"
            assert len(self.blend_per_split) == len(Split), f"blend_per_split must contain {len(Split)} blends"
            if self.split is not None:
                self.split = None
                log_rank_0(logging.WARNING, "Let split = None")
        elif self.blend is not None:
            assert self.split is not None, "both blend and split must be provided"
            self.split_vector = _parse_and_normalize_split(self.split)
            log_rank_0(logging.INFO, f"Let split_vector = {self.split_vector}")


@dataclass
class GPTDatasetConfig(BlendedMegatronDatasetConfig):
    return_document_ids: bool = False
    fim_rate: float = 0
    fim_spm_rate: float = 0


def _parse_and_normalize_split(split: str) -> list[float]:
    values = [float(v) for v in re.findall(r"[.0-9]+", split)]
    values += [0.0] * (len(Split) - len(values))
    assert len(values) == len(Split) and all(v >= 0 for v in values)
    return normalize(values)


# ----------------------------------------------------------------------------------------------------------------------
class BlendedDataset(torch.utils.data.Dataset):
    """``size`` samples interleaved from ``datasets`` so that every prefix of the order matches ``weights`` as closely
    as possible."""

    def __init__(self, datasets: list, weights: list[float], size: int, config: BlendedMegatronDatasetConfig,
                 caching_allowed: bool) -> None:
        assert len(datasets) < np.iinfo(np.int16).max
        assert len(datasets) == len(weights)
        assert np.isclose(sum(weights), 1.0)
        assert all(type(d) == type(datasets[0]) for d in datasets)
        if len(datasets) == 1:
            log_rank_0(logging.WARNING, "Building a BlendedDataset for a single MegatronDataset")
        self.datasets = datasets
        self.weights = normalize(weights)  # again, to stay bitwise identical to Megatron-LM
        self.size = size
        self.config = config
        self.caching_allowed = caching_allowed

        ids = OrderedDict()
        ids["class"] = type(self).__name__
        ids["datasets"] = [d.unique_identifiers for d in datasets]
        ids["weights"] = self.weights
        ids["size"] = size
        self.unique_description = json.dumps(ids, indent=4)
        self.unique_description_hash = hashlib.md5(self.unique_description.encode("utf-8")).hexdigest()

        self.dataset_index, self.dataset_sample_index = self._build_indices()
        _ = self[size - 1]  # the last sample must exist in its dataset ...
        try:
            _ = self[size]  # ... and the index arrays must end there
        except IndexError:
            log_rank_0(logging.INFO, f"> {type(self).__name__} length: {len(self)}")
        else:
            raise RuntimeError(f"{type(self).__name__} size is improperly bounded")

    def __len__(self) -> int:
        return self.size

    def __getitem__(self, idx: int) -> dict:
        dataset_id = self.dataset_index[idx]
        return {"dataset_id": dataset_id, **self.datasets[dataset_id][self.dataset_sample_index[idx]]}

    def _build_indices(self) -> tuple[np.ndarray, np.ndarray]:
        cache_dir = self.config.path_to_cache
        paths, cache_hit = None, False
        if cache_dir:
            stem = os.path.join(cache_dir, f"{self.unique_description_hash}-{type(self).__name__}-")
            paths = {k: stem + k for k in ("description.txt", "dataset_index.npy", "dataset_sample_index.npy")}
            cache_hit = all(os.path.isfile(p) for p in paths.values())

        if not cache_dir or (not cache_hit and self.caching_allowed):
            log_rank_0(logging.INFO, f"Build and save the {type(self).__name__} indices")
            dataset_index = np.zeros(self.size, dtype=np.int16)
            dataset_sample_index = np.zeros(self.size, dtype=np.int64)
            build_blending_indices(dataset_index, dataset_sample_index, self.weights, len(self.datasets), self.size, False)
            if cache_dir:
                os.makedirs(cache_dir, exist_ok=True)
                with open(paths["description.txt"], "wt") as f:
                    f.write(self.unique_description)
                np.save(paths["dataset_index.npy"], dataset_index, allow_pickle=True)
                np.save(paths["dataset_sample_index.npy"], dataset_sample_index, allow_pickle=True)
            else:
                log_rank_0(logging.WARNING, "Unable to save the indexes because path_to_cache is None")
            return dataset_index, dataset_sample_index

        log_rank_0(logging.INFO, f"Load the {type(self).__name__} indices")
        return (np.load(paths["dataset_index.npy"], allow_pickle=True, mmap_mode="r"),
                np.load(paths["dataset_sample_index.npy"], allow_pickle=True, mmap_mode="r"))


# ----------------------------------------------------------------------------------------------------------------------
def _split_bounds(split: list[float], num_elements: int) -> list[int]:
    """Element ranges of the splits, e.g. ``[0, 900, 990, 1000]`` for 1000 elements split 90/9/1; the rounding error
    is taken off every bound so that the last one is exactly ``num_elements``."""
    bounds = [0]
    for fraction in split:
        bounds.append(bounds[-1] + int(round(fraction * float(num_elements))))
    excess = bounds[-1] - num_elements
    bounds[1:] = [b - excess for b in bounds[1:]]
    assert bounds[-1] == num_elements
    return bounds


def _blend_prefixes_weights_sizes(blend: list, target_samples_per_split: list[int]):
    """Per store: prefix, normalised weight and the number of samples to request per split (0.5 % head-room so that
    the blended order never runs a store dry)."""
    weights = normalize([float(blend[i]) for i in range(0, len(blend), 2)])
    prefixes = [str(blend[i + 1]).strip() for i in range(0, len(blend), 2)]
    sizes = [[int(math.ceil(target * w * 1.005)) for target in target_samples_per_split] for w in weights]
    return prefixes, weights, sizes


def _index_dtype(bounds: list[int]):
    top = max(bounds)
    if top <= np.iinfo(np.int32).max:
        return np.int32
    if top <= np.iinfo(np.int64).max:
        return np.int64
    raise ValueError("value for split idx is too large")


class BlendedMegatronDatasetBuilder:
    """Builds train/valid/test datasets (plain or blended) on the ranks that should hold them.

    With ``torch.distributed`` initialised, global rank 0 (and local rank 0 of every node when
    ``node_uses_local_storage``) builds first and writes the index caches; after a barrier the other building ranks
    construct the same datasets from the caches. Ranks with ``is_built_on_rank=False`` get ``None``."""

    def __init__(self, cls, sizes: list[int], config: BlendedMegatronDatasetConfig, tokenizer) -> None:
        self.cls = cls
        self.sizes = sizes
        self.config = config
        self.tokenizer = tokenizer

    # -- one distribution split three ways, or one distribution per split ------------------------------------------------
    def build(self) -> list:
        if self.config.blend:
            blend, split = self.config.blend, self.config.split_vector
            if len(blend) == 1:
                return self._build_splits(blend[0], split, self.sizes)
            prefixes, weights, sizes = _blend_prefixes_weights_sizes(blend, self.sizes)
            per_split = [[] for _ in Split]
            for prefix, size in zip(prefixes, sizes):
                for j, dataset in enumerate(self._build_splits(prefix, split, size)):
                    per_split[j].append(dataset)
            totals = [sum(column) for column in zip(*sizes)]
            out = []
            for j in range(len(Split)):
                missing = [d is None for d in per_split[j]]
                if split[j] == 0.0:
                    assert all(missing)
                    out.append(None)
                else:
                    assert all(missing) or not any(missing)
                    out.append(self._construct(BlendedDataset, datasets=per_split[j], weights=weights, size=totals[j], config=self.config))
            return out

        out = []
        for j in range(len(Split)):
            blend = self.config.blend_per_split[j]
            if not blend:
                out.append(None)
                continue
            split = [0.0] * len(Split)
            split[j] = 1.0
            sizes = [0] * len(Split)
            sizes[j] = self.sizes[j]
            if len(blend) == 1:
                out.append(self._build_splits(blend[0], split, sizes)[j])
                continue
            prefixes, weights, per_store = _blend_prefixes_weights_sizes(blend, sizes)
            datasets = [self._build_splits(prefix, split, size)[j] for prefix, size in zip(prefixes, per_store)]
            totals = [sum(column) for column in zip(*per_store)]
            out.append(self._construct(BlendedDataset, datasets=datasets, weights=weights, size=totals[j], config=self.config))
        return out

    def _build_splits(self, path_prefix: str, split: list[float], sizes: list[int]) -> list:
        store = self._open_store(path_prefix)
        indices = [None] * len(Split)
        if store is not None:
            count = store.sequence_lengths.shape[0] if self.cls.is_split_by_sequence() else store.document_indices.shape[0] - 1
            bounds = _split_bounds(split, count)
            dtype = _index_dtype(bounds)
            indices = [np.arange(bounds[j], bounds[j + 1], dtype=dtype) for j in range(len(Split))]
        out = []
        for j, which in enumerate(Split):
            if split[j] == 0.0:
                out.append(None)
            else:
                out.append(self._construct(self.cls, indexed_dataset=store, indexed_indices=indices[j], num_samples=sizes[j],
                                           index_split=which, tokenizer=self.tokenizer, config=self.config))
        return out

    # -- named groups of (path, "start:end" fraction range, weight) for one split ------------------------------------------
    def build_dataset_single_split(self, group_names, split_paths, split_splits, split_weights, data_split: Split) -> list:
        j = data_split.value
        assert len(split_paths) == len(group_names) == len(split_splits) == len(split_weights)
        out = []
        for names, paths, ranges, weights in zip(group_names, split_paths, split_splits, split_weights):
            assert len(paths) == len(ranges) == len(weights)
            if len(paths) == 1:
                assert weights[0] == 1
                out.append(self._build_range(names[0], paths[0], ranges[0], self.sizes[j], data_split))
                continue
            blend = [v for pair in zip(weights, paths) for v in pair]
            _, normalised, sizes = _blend_prefixes_weights_sizes(blend, self.sizes)
            datasets = [self._build_range(n, p, r, s[j], data_split) for n, p, r, s in zip(names, paths, ranges, sizes)]
            totals = [sum(column) for column in zip(*sizes)]
            out.append(self._construct(BlendedDataset, datasets=datasets, weights=normalised, size=totals[j], config=self.config))
        return out

    def _build_range(self, group_name: str, path_prefix: str, fraction_range: str, size: int, data_split: Split):
        store = self._open_store(path_prefix)
        start, end = (float(v) for v in fraction_range.split(":"))
        config = deepcopy(self.config)
        config.name = group_name
        config.split = fraction_range
        indices = None
        if store is not None:
            count = store.sequence_lengths.shape[0] if self.cls.is_split_by_sequence() else store.document_indices.shape[0] - 1
            start, end = int(start * count), int(end * count)
            indices = np.arange(start, end, dtype=_index_dtype([start, end]))
        if start == end:
            return None
        return self._construct(self.cls, indexed_dataset=store, indexed_indices=indices, num_samples=size, index_split=data_split,
                               tokenizer=self.tokenizer, config=config)

    # ------------------------------------------------------------------------------------------------------------------
    def _construct(self, cls, **kwargs):
        if not torch.distributed.is_initialized():
            return cls(**kwargs, caching_allowed=True)
        local_first = ProcessGroupManager.get_local_rank() == 0
        writer = ProcessGroupManager.get_global_rank() == 0 or (local_first and self.config.node_uses_local_storage)
        dataset = None
        if writer and self.config.is_built_on_rank:
            try:
                dataset = cls(**kwargs, caching_allowed=True)
            except OSError as err:
                raise Exception("Failed to write dataset materials to the data cache directory. Please supply a directory to which "
                                "you have write access via the path_to_cache attribute in BlendedMegatronDatasetConfig and retry.") from err
        torch.distributed.barrier()
        if not writer and self.config.is_built_on_rank:
            dataset = cls(**kwargs, caching_allowed=False)
        return dataset

    def _open_store(self, path_prefix: str):
        if not torch.distributed.is_initialized() or self.config.is_built_on_rank:
            return MMapIndexedDataset(path_prefix, self.cls.is_multimodal())
        return None

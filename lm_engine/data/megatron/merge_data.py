"""Concatenate token stores without re-tokenising (parity: lm_engine/data/megatron/merge_data.py:9-17)."""

from __future__ import annotations

from .indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder, get_bin_path, get_idx_path


def merge_files(input_prefixes: list[str], output_prefix: str) -> None:
    dtype = MMapIndexedDataset(input_prefixes[0]).index.dtype
    builder = MMapIndexedDatasetBuilder(get_bin_path(output_prefix), dtype=dtype)
    for prefix in input_prefixes:
        builder.add_index(prefix)
    builder.finalize(get_idx_path(output_prefix))

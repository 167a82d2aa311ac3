"""Shared pieces of the Megatron-format data stack: split enum, weight normalisation and the native index builders.

Parity: lm_engine/data/megatron/utils/__init__.py:14-82. The index builders are C++ functions of the engine's
extension (``csrc/data/helpers.cpp``), which is compiled ahead of time with everything else instead of at first use;
plain NumPy/Python versions with identical results serve machines without the built extension.
"""

from __future__ import annotations

from enum import Enum

import numpy as np


class Split(Enum):
    train = 0
    valid = 1
    test = 2


def compile_helpers() -> None:
    """Kept for API parity: the helpers are part of the ahead-of-time extension build, so there is nothing to do."""


def _helpers():
    try:
        from ...ops.build import load_extension

        return load_extension(build_if_missing=False)
    except Exception:
        return None


def normalize(weights: list[float]) -> list[float]:
    w = np.asarray(weights, dtype=np.float64)
    return (w / w.sum()).tolist()


def build_blending_indices(dataset_index: np.ndarray, dataset_sample_index: np.ndarray, weights: list[float],
                           num_datasets: int, size: int, verbose: bool = False) -> None:
    """Fill ``dataset_index`` (int16) / ``dataset_sample_index`` (int64): sample ``i`` goes to the dataset whose count
    lags its target ``weight * (i + 1)`` the most (first one on ties)."""
    native = _helpers()
    if native is not None:
        native.build_blending_indices(dataset_index, dataset_sample_index, np.asarray(weights, dtype=np.float64), num_datasets, size, verbose)
        return
    w = np.asarray(weights, dtype=np.float64)
    taken = np.zeros(num_datasets, dtype=np.int64)
    for i in range(size):
        denominator = max(float(i), 1.0)
        errors = w * denominator - taken
        pick = int(np.argmax(errors))
        dataset_index[i] = pick
        dataset_sample_index[i] = taken[pick]
        taken[pick] += 1


def build_sample_idx(sizes: np.ndarray, doc_idx: np.ndarray, sequence_length: int, num_epochs: int,
                     tokens_per_epoch: int) -> np.ndarray:
    """``[num_samples + 1, 2]`` array of (position in ``doc_idx``, token offset) marking where each sample of
    ``sequence_length + 1`` tokens starts; consecutive samples overlap by one token."""
    if doc_idx.dtype not in (np.int32, np.int64):
        raise ValueError("unexpected dtype for doc_idx")
    native = _helpers()
    if native is not None:
        fn = native.build_sample_idx_int32 if doc_idx.dtype == np.int32 else native.build_sample_idx_int64
        return fn(np.ascontiguousarray(sizes, dtype=np.int32), np.ascontiguousarray(doc_idx), sequence_length, num_epochs, int(tokens_per_epoch))

    num_samples = (num_epochs * int(tokens_per_epoch) - 1) // sequence_length
    out = np.zeros((num_samples + 1, 2), dtype=doc_idx.dtype)
    position, offset = 0, 0
    for sample in range(1, num_samples + 1):
        remaining = sequence_length + 1
        while remaining != 0:
            available = int(sizes[doc_idx[position]]) - offset
            remaining -= available
            if remaining <= 0:
                offset += remaining + available - 1
                remaining = 0
            else:
                position += 1
                offset = 0
        out[sample, 0], out[sample, 1] = position, offset
    return out

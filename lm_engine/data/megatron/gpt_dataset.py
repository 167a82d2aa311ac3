"""GPT pretraining dataset over a token store: fixed-length samples cut from a shuffled stream of documents.

Parity: lm_engine/data/megatron/gpt_dataset.py:23-578 and megatron_dataset.py:15-131. Index construction consumes the
NumPy ``RandomState`` in the same order (document shuffle, then sample shuffle), and the cache file names are built from
the same description hash, so indices cached by either implementation are interchangeable.

Three indices define the data order:
  document index  the exposed documents repeated for every epoch and shuffled (last epoch shuffled separately when
                  less than 80 % of it is needed, so it does not dilute the earlier epochs);
  sample index    ``[num_samples + 1, 2]`` (position in the document index, token offset) of every sample start;
                  sample ``i`` is the ``sequence_length + 1`` tokens from start ``i`` to start ``i + 1`` inclusive;
  shuffle index   permutation applied to the sample number.
"""

from __future__ import annotations

import hashlib
import json
import logging
import os
from collections import OrderedDict

import numpy as np
import torch

from ...utils import log_rank_0
from .indexed_dataset import MMapIndexedDataset
from .utils import Split, build_sample_idx

FIM_PREFIX, FIM_MIDDLE, FIM_SUFFIX, FIM_PAD = "<fim_prefix>", "<fim_middle>", "<fim_suffix>", "<fim_pad>"
_FINAL_EPOCH_THRESHOLD = 0.80


class MegatronDataset(torch.utils.data.Dataset):
    """Base: a view of ``indexed_indices`` of a token store from which ``num_samples`` samples are drawn."""

    def __init__(self, indexed_dataset: MMapIndexedDataset, indexed_indices: np.ndarray, num_samples: int,
                 index_split: Split, config, caching_allowed: bool) -> None:
        assert indexed_indices.size > 0 and num_samples > 0
        assert self.is_multimodal() == indexed_dataset.multimodal
        self.indexed_dataset = indexed_dataset
        self.indexed_indices = indexed_indices
        self.num_samples = num_samples
        self.index_split = index_split
        self.config = config
        self.caching_allowed = caching_allowed

        ids = OrderedDict()
        ids["class"] = type(self).__name__
        ids["path_prefix"] = indexed_dataset.path_prefix
        ids["num_samples"] = num_samples
        ids["index_split"] = index_split.name
        for name in self._key_config_attributes():
            ids[name] = getattr(config, name)
        self.unique_identifiers = ids
        self.unique_description = json.dumps(ids, indent=4)
        self.unique_description_hash = hashlib.md5(self.unique_description.encode("utf-8")).hexdigest()
        self._finalize()

    def _finalize(self) -> None:
        raise NotImplementedError

    @staticmethod
    def is_multimodal() -> bool:
        return False

    @staticmethod
    def is_split_by_sequence() -> bool:
        return True

    @classmethod
    def is_split_by_document(cls) -> bool:
        return not cls.is_split_by_sequence()

    @staticmethod
    def _key_config_attributes() -> list[str]:
        return ["name", "split", "random_seed", "sequence_length"]


def _epochs_needed(tokens_per_epoch: int, sequence_length: int, num_samples: int) -> int:
    # a sample takes sequence_length + 1 tokens but shares its last token with the next one
    epochs = 1
    while (epochs * tokens_per_epoch - 1) // sequence_length < num_samples:
        epochs += 1
    return epochs


def _build_document_index(documents: np.ndarray, num_epochs: int, rng: np.random.RandomState, separate_final_epoch: bool) -> np.ndarray:
    if separate_final_epoch and num_epochs > 1:
        head = _build_document_index(documents, num_epochs - 1, rng, False)
        tail = _build_document_index(documents, 1, rng, False)
        return np.concatenate((head, tail))
    index = np.tile(documents, num_epochs).astype(documents.dtype)
    rng.shuffle(index)
    return index


def _build_shuffle_index(num_samples: int, total_size: int, rng: np.random.RandomState) -> np.ndarray:
    dtype = np.uint32 if total_size < np.iinfo(np.uint32).max - 1 else np.int64
    first = np.arange(num_samples, dtype=dtype)
    rng.shuffle(first)
    if num_samples == total_size:
        return first
    last = np.arange(num_samples, total_size, dtype=dtype)
    rng.shuffle(last)
    return np.concatenate((first, last))


class GPTDataset(MegatronDataset):
    def __init__(self, indexed_dataset, indexed_indices, num_samples, index_split, tokenizer, config, caching_allowed) -> None:
        self.tokenizer = tokenizer
        self.fim_rate = config.fim_rate
        self.fim_spm_rate = config.fim_spm_rate
        self.np_rng = np.random.RandomState(seed=config.random_seed)  # consumed only by fill-in-the-middle
        if self.fim_rate != 0:
            assert 0 <= self.fim_rate <= 1, "FIM rate must be a probability 0 <= rate <= 1"
            self.suffix_tok_id, self.prefix_tok_id, self.middle_tok_id, self.pad_tok_id = (
                tokenizer.convert_tokens_to_ids(t) for t in (FIM_SUFFIX, FIM_PREFIX, FIM_MIDDLE, FIM_PAD))
        super().__init__(indexed_dataset, indexed_indices, num_samples, index_split, config, caching_allowed)

    def _finalize(self) -> None:
        self.document_index, self.sample_index, self.shuffle_index = self._build_document_sample_shuffle_indices()

    def __len__(self) -> int:
        return self.sample_index.shape[0] - 1

    def __getitem__(self, idx: int) -> dict[str, np.ndarray]:
        text, document_ids = self._query_document_sample_shuffle_indices(idx)
        if self.config.return_document_ids:
            return {"text": text, "document_ids": document_ids}
        return {"text": text}

    # ------------------------------------------------------------------------------------------------------------------
    def _query_document_sample_shuffle_indices(self, idx: int) -> tuple[np.ndarray, np.ndarray]:
        idx = self.shuffle_index[idx]
        first, first_offset = self.sample_index[idx]
        last, last_offset = self.sample_index[idx + 1]
        store = self.indexed_dataset
        documents = [self.document_index[i] for i in range(first, last + 1)]
        if first == last:
            parts = [store.get(documents[0], offset=first_offset, length=last_offset - first_offset + 1)]
        else:
            parts = [store.get(documents[0], offset=first_offset)]
            parts += [store.get(d) for d in documents[1:-1]]
            parts.append(store.get(documents[-1], length=last_offset + 1))
        sample = np.array(np.concatenate(parts), dtype=np.int64)
        if self.fim_rate != 0:
            sample = self._fill_in_the_middle(sample)
        return sample, np.array(documents, dtype=np.int64)

    def _fill_in_the_middle(self, sample: np.ndarray) -> np.ndarray:
        """Apply the FIM transformation independently to every document fragment of the sample (fragments are
        separated by the end-of-document token), then cut or pad back to the original length."""
        length = sample.shape[0]
        eod = self.tokenizer.eod
        breaks = np.flatnonzero(sample == eod)
        pieces, start = [], 0
        for stop in breaks:
            if stop > start:
                pieces += [self._permute(sample[start:stop]), [eod]]
            start = stop + 1
        if breaks.size == 0:
            pieces = [self._permute(sample)]
        else:
            pieces.append(self._permute(sample[start:]))
        sample = np.concatenate(pieces)
        if sample.shape[0] > length:
            sample = sample[:length]
        elif sample.shape[0] < length:
            sample = np.concatenate([sample, np.full(length - sample.shape[0], self.pad_tok_id)])
        return sample

    def _permute(self, fragment: np.ndarray) -> np.ndarray:
        permuted, self.np_rng = permute(fragment, self.np_rng, self.fim_rate, self.fim_spm_rate, self.tokenizer, truncate_or_pad=False,
                                        suffix_tok_id=self.suffix_tok_id, prefix_tok_id=self.prefix_tok_id,
                                        middle_tok_id=self.middle_tok_id, pad_tok_id=self.pad_tok_id)
        return permuted

    # ------------------------------------------------------------------------------------------------------------------
    def _build_document_sample_shuffle_indices(self) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
        cache_dir = self.config.path_to_cache
        if cache_dir is None:
            cache_dir = os.path.join(self.indexed_dataset.path_prefix, "cache", f"{type(self).__name__}_indices")
        stem = os.path.join(cache_dir, f"{self.unique_description_hash}-{type(self).__name__}-")
        paths = {k: stem + k for k in ("description.txt", "document_index.npy", "sample_index.npy", "shuffle_index.npy")}
        cache_hit = all(os.path.isfile(p) for p in paths.values())

        sequence_length = self.config.sequence_length
        tokens_per_epoch = int(np.sum(self.indexed_dataset.sequence_lengths[self.indexed_indices]))
        num_epochs = _epochs_needed(tokens_per_epoch, sequence_length, self.num_samples)
        log_rank_0(logging.INFO, f"> Tokens per epoch: {tokens_per_epoch}")
        log_rank_0(logging.INFO, f"> Number of epochs: {num_epochs}")

        if not cache_hit and self.caching_allowed:
            log_rank_0(logging.INFO, f"Build and save the {type(self).__name__} {self.index_split.name} indices")
            separate_final_epoch = False
            samples_before_final = 0
            if num_epochs > 1:
                samples_before_final = ((num_epochs - 1) * tokens_per_epoch - 1) // sequence_length
                from_final = self.num_samples - samples_before_final
                per_epoch = (tokens_per_epoch - 1) // sequence_length
                assert 0 <= from_final <= per_epoch + 1
                separate_final_epoch = from_final < int(_FINAL_EPOCH_THRESHOLD * per_epoch)

            rng = np.random.RandomState(self.config.random_seed)
            os.makedirs(cache_dir, exist_ok=True)
            with open(paths["description.txt"], "wt") as f:
                f.write(self.unique_description)

            document_index = _build_document_index(self.indexed_indices, num_epochs, rng, separate_final_epoch)
            np.save(paths["document_index.npy"], document_index, allow_pickle=True)

            assert self.indexed_dataset.sequence_lengths.dtype == np.int32
            sample_index = build_sample_idx(self.indexed_dataset.sequence_lengths, document_index, sequence_length, num_epochs, tokens_per_epoch)
            np.save(paths["sample_index.npy"], sample_index, allow_pickle=True)

            total = sample_index.shape[0] - 1
            shuffle_index = _build_shuffle_index(samples_before_final if separate_final_epoch else total, total, rng)
            np.save(paths["shuffle_index.npy"], shuffle_index, allow_pickle=True)

        log_rank_0(logging.INFO, f"Load the {type(self).__name__} {self.index_split.name} indices")
        document_index = np.load(paths["document_index.npy"], allow_pickle=True, mmap_mode="r")
        sample_index = np.load(paths["sample_index.npy"], allow_pickle=True, mmap_mode="r")
        shuffle_index = np.load(paths["shuffle_index.npy"], allow_pickle=True, mmap_mode="r")
        log_rank_0(logging.INFO, f"> total number of samples: {sample_index.shape[0] - 1}")
        log_rank_0(logging.INFO, f"> total number of epochs: {num_epochs}")
        return document_index, sample_index, shuffle_index


def permute(sample: np.ndarray, np_rng: np.random.RandomState, fim_rate: float, fim_spm_rate: float, tokenizer,
            truncate_or_pad: bool = True, suffix_tok_id: int | None = None, prefix_tok_id: int | None = None,
            middle_tok_id: int | None = None, pad_tok_id: int | None = None):
    """With probability ``fim_rate`` split the decoded text at two random character positions and re-emit it as
    prefix/suffix/middle with sentinel tokens (PSM order, or SPM with probability ``fim_spm_rate``)."""
    if not np_rng.binomial(1, fim_rate):
        return sample, np_rng
    contents = tokenizer.detokenize(sample)
    lo, hi = sorted(np_rng.randint(low=0, high=len(contents) + 1, size=2))
    prefix = np.array([*tokenizer.tokenize(contents[:lo])], dtype=np.int64)
    middle = np.array([*tokenizer.tokenize(contents[lo:hi])], dtype=np.int64)
    suffix = np.array([*tokenizer.tokenize(contents[hi:])], dtype=np.int64)
    if truncate_or_pad:
        diff = suffix.shape[0] + prefix.shape[0] + middle.shape[0] + 3 - sample.shape[0]
        if diff > 0:
            if suffix.shape[0] <= diff:
                return sample, np_rng
            suffix = suffix[: suffix.shape[0] - diff]
        elif diff < 0:
            suffix = np.concatenate([suffix, np.full(-diff, pad_tok_id)])
    if np_rng.binomial(1, fim_spm_rate):
        out = np.concatenate([[prefix_tok_id, suffix_tok_id], suffix, [middle_tok_id], prefix, middle])
    else:
        out = np.concatenate([[prefix_tok_id], prefix, [suffix_tok_id], suffix, [middle_tok_id], middle])
    return out, np_rng

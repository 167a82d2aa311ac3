"""Data layer entry points (parity: lm_engine/data/__init__.py:37-325)."""

from __future__ import annotations

import logging
from typing import Iterable

import torch

from ..enums import DatasetSplit, Mode
from ..utils import ProcessGroupManager, log_rank_0
from .synthetic import SyntheticTokenLoader


def get_next_batch(dataloader: Iterable | None) -> dict | None:
    """Next batch, or None on ranks that do not read data themselves (non-source tensor parallel ranks)."""
    if dataloader is None:
        return None
    return next(dataloader)


def custom_iterator(x: Iterable | None, infinite: bool):
    """Iterate once or forever over ``x`` (None stays None)."""
    if x is None:
        return None

    def forever():
        while True:
            for item in x:
                yield item

    def once():
        for item in x:
            yield item

    return forever() if infinite else once()


def get_pretraining_dataloaders(args, tokenizer, consumed_samples: int):
    """Returns ``(train_iterator, val_iterators, test_iterators)`` for the dataset class named in the config."""
    if len(args.datasets) != 1:
        raise ValueError("pretraining expects exactly one dataset entry")
    class_name = args.datasets[0].class_name
    if class_name == "SyntheticDataset":
        return _get_synthetic_dataloaders(args, consumed_samples)
    if class_name == "MegatronDataset":
        from .megatron import get_megatron_gpt_dataloaders

        return get_megatron_gpt_dataloaders(args, tokenizer, consumed_samples=consumed_samples)
    if class_name in ("IBMDataset", "FSDPDataset"):
        from .ibm import get_ibm_dataloaders

        return get_ibm_dataloaders(args, tokenizer)
    raise ValueError(f"unexpected dataset class for pretraining ({class_name})")


def _get_synthetic_dataloaders(args, consumed_samples: int):
    class_args = args.datasets[0].class_args
    config = args.model_args.pretrained_config or {}
    vocab_size = class_args.get("vocab_size", config.get("vocab_size"))
    if vocab_size is None:
        raise ValueError("SyntheticDataset needs class_args.vocab_size (or a pretrained_config with vocab_size)")
    loader = SyntheticTokenLoader(
        vocab_size=vocab_size,
        sequence_length=class_args["sequence_length"],
        micro_batch_size=args.training_parameters.micro_batch_size,
        seed=class_args.get("seed", args.random_args.seed),
        dp_rank=ProcessGroupManager.get_data_parallel_rank(),
        dp_world_size=ProcessGroupManager.get_data_parallel_world_size(),
        pin_memory=class_args.get("pin_memory", True),
    )
    loader.set_consumed_samples(consumed_samples)
    log_rank_0(logging.INFO, "using synthetic uniform-random tokens")
    return loader, [], []


def __getattr__(name: str):
    import importlib

    lazy = {
        "get_megatron_gpt_dataloaders": ".megatron", "get_finetuning_dataloader": ".finetuning",
        "get_datasets_list": ".finetuning", "collate_fn": ".utils", "BlendedDatasets": ".base", "BaseDataset": ".base",
        "BlendedDistributedSampler": ".sampler", "ResumableDataLoader": ".dataloader",
        "DispatchingDataLoader": ".dataloader", "AlpacaDataset": ".instruction_tuning", "DollyDataset": ".instruction_tuning",
        "SlimOrcaDataset": ".instruction_tuning", "DebugDataset": ".debug", "HuggingFaceDataset": ".huggingface",
        "SST2Dataset": ".sst2", "get_ibm_dataloaders": ".ibm",
    }
    if name in lazy:
        return getattr(importlib.import_module(lazy[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

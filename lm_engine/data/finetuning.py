"""Factories for finetuning / inference dataloaders (parity: lm_engine/data/__init__.py:37-135)."""

from __future__ import annotations

import logging
from functools import partial

from ..enums import DatasetSplit, Mode
from ..utils import ProcessGroupManager, log_rank_0
from .base import BaseDataset, BlendedDatasets
from .dataloader import ResumableDataLoader
from .debug import DebugDataset
from .huggingface import HuggingFaceDataset
from .instruction_tuning import AlpacaDataset, DollyDataset, SlimOrcaDataset
from .sampler import BlendedDistributedSampler
from .sst2 import SST2Dataset
from .utils import collate_fn

_FINETUNING_DATASETS = {
    "AlpacaDataset": AlpacaDataset, "DebugDataset": DebugDataset, "DollyDataset": DollyDataset,
    "HuggingFaceDataset": HuggingFaceDataset, "SlimOrcaDataset": SlimOrcaDataset, "SST2Dataset": SST2Dataset,
}


def get_datasets_list(dataset_args_list, split: DatasetSplit, mode: Mode, tokenizer, is_encoder_decoder: bool):
    """Instantiate every configured dataset for ``split``; returns ``(non-empty datasets, their sampling ratios)``."""
    datasets, ratios = [], []
    for data_args in dataset_args_list:
        if data_args.class_name not in _FINETUNING_DATASETS:
            raise ValueError(f"invalid class_name ({data_args.class_name}) for dataset")
        dataset = _FINETUNING_DATASETS[data_args.class_name](
            class_args=data_args.class_args, split=split, mode=mode, tokenizer=tokenizer, is_encoder_decoder=is_encoder_decoder,
            data_name=data_args.data_name, input_format=data_args.input_format, output_format=data_args.output_format,
            max_input_tokens=data_args.max_input_tokens, max_output_tokens=data_args.max_output_tokens)
        if len(dataset) > 0:
            datasets.append(dataset)
            ratios.append(data_args.data_sampling_ratio)
            log_rank_0(logging.INFO, f"examples in {type(dataset).__name__} ({data_args.data_name}) = {len(dataset)}")
    ratios = [1 if r is None else r for r in ratios]
    return datasets, ratios


def get_finetuning_dataloader(args, split: DatasetSplit, mode: Mode, tokenizer, is_encoder_decoder: bool):
    """Only the first tensor parallel rank builds a loader (the others receive broadcast batches): returns None there."""
    if not ProcessGroupManager.is_tensor_parallel_first_rank():
        return None
    datasets, ratios = get_datasets_list(args.datasets, split, mode, tokenizer, is_encoder_decoder)
    if len(datasets) == 0:
        return None
    blended = BlendedDatasets(datasets, split)
    training = mode == Mode.training
    sampler = BlendedDistributedSampler(
        dataset=blended, data_sampling_ratios=ratios, num_replicas=ProcessGroupManager.get_data_parallel_world_size(),
        rank=ProcessGroupManager.get_data_parallel_rank(),
        ignore_sampling_proportion_for_validation=getattr(args.training_parameters, "ignore_sampling_proportion_for_validation", True) if training else True,
        shuffle=split == DatasetSplit.train, seed=args.random_args.seed, drop_last=False)
    batch_size = args.training_parameters.micro_batch_size if training else args.generation_parameters.batch_size
    use_padding_free = args.model_args.use_padding_free_transformer if args.model_args is not None else False
    tp = ProcessGroupManager.get_tensor_parallel_world_size()
    collate = partial(
        collate_fn, mode=mode, loss_mask=args.training_parameters.loss_mask if training else None,
        eos_token_id=tokenizer.eos_token_id, is_encoder_decoder=is_encoder_decoder,
        use_padding_free_transformer=use_padding_free, pad_to_multiple_of=tp if use_padding_free else 1,
        device=ProcessGroupManager.get_device())
    loader = ResumableDataLoader(blended, batch_size=batch_size, sampler=sampler, collate_fn=collate, drop_last=False)
    log_rank_0(logging.INFO, f"{'*' * 25} {split.value} {'*' * 25}")
    log_rank_0(logging.INFO, str(blended))
    if training:
        log_rank_0(logging.INFO, str(sampler))
    return loader

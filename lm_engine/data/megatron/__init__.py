"""Pretraining dataloaders over Megatron-format token stores.

Parity: lm_engine/data/megatron/__init__.py:18-243. ``class_args`` of the single dataset entry select one of:
``data_path`` (one prefix, or weight/prefix pairs, split by ``split``), ``train_data_path`` / ``val_data_path`` /
``test_data_path`` (one blend per split), or ``train_weighted_split_paths`` (+ ``val_`` / ``test_``) groups of
``{path, split: "start:end", weight}``.

Data order equals Megatron-LM's: sample numbers are dealt in global micro-batches to the data parallel ranks, so a run
resumes by passing ``consumed_samples``. With the dispatching dataloader only the first rank of every node reads the
store and broadcasts the node's micro-batches inside the node.
"""

from __future__ import annotations

import logging

import torch
import torch.distributed as dist

from ...defaults import INPUT_FORMAT, OUTPUT_FORMAT
from ...utils import ProcessGroupManager, log_rank_0
from ..dataloader import DispatchingDataLoader, ResumableDataLoader
from .blended import BlendedDataset, BlendedMegatronDatasetBuilder, BlendedMegatronDatasetConfig, GPTDatasetConfig
from .gpt_dataset import GPTDataset, MegatronDataset
from .indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder
from .sampler import MegatronBatchSampler
from .utils import Split, compile_helpers


def _train_val_test_samples(num_training_steps: int, micro_batch_size: int, gradient_accumulation_steps: int,
                            eval_interval: int | None, eval_steps: int | None) -> tuple[int, int, int]:
    per_step = micro_batch_size * gradient_accumulation_steps * ProcessGroupManager.get_data_parallel_world_size()
    eval_steps = eval_steps or 0
    evaluations = num_training_steps // eval_interval + 1 if eval_interval else 1
    return num_training_steps * per_step, evaluations * eval_steps * per_step, eval_steps * per_step


def _node_broadcast_groups(ranks_per_node: int) -> dict[int, dist.ProcessGroup]:
    """{first rank of node: group of the node's ranks}; every rank creates every group (collective call)."""
    world = ProcessGroupManager.get_world_size()
    return {first: dist.new_group(list(range(first, min(first + ranks_per_node, world)))) for first in range(0, world, ranks_per_node)}


def get_megatron_gpt_dataloaders(args, tokenizer, consumed_samples: int):
    assert len(args.datasets) == 1
    entry = args.datasets[0]
    class_args = entry.class_args
    assert entry.max_input_tokens is None and entry.max_output_tokens is None
    assert entry.input_format == INPUT_FORMAT and entry.output_format == OUTPUT_FORMAT

    micro_batch_size = args.training_parameters.micro_batch_size
    accumulation = args.training_parameters.gradient_accumulation_steps
    pipeline_stages = args.distributed_args.num_pipeline_stages
    sequence_length = class_args.get("sequence_length")
    # with pipeline parallelism the first stage pulls all micro-batches of a step in one go
    samples_per_fetch = micro_batch_size if pipeline_stages == 1 else micro_batch_size * accumulation
    num_workers = class_args.get("num_workers", 2)
    dispatching = args.distributed_args.dispatching_dataloader

    compile_helpers()
    log_rank_0(logging.INFO, "> building train, validation, and test datasets for GPT ...")

    if dispatching:
        assert ProcessGroupManager.get_tensor_parallel_world_size() == 1, "tensor parallel doesn't support dispatching dataloader"
        ranks_per_node = max(torch.cuda.device_count(), 1) if torch.cuda.is_available() else class_args.get("ranks_per_node", ProcessGroupManager.get_world_size())
        ranks_per_node = min(ranks_per_node, ProcessGroupManager.get_world_size())
        node_rank = ProcessGroupManager.get_global_rank() // ranks_per_node
        num_nodes = ProcessGroupManager.get_world_size() // ranks_per_node
        groups = _node_broadcast_groups(ranks_per_node)
        source_rank = node_rank * ranks_per_node
        is_built_on_rank = ProcessGroupManager.get_global_rank() == source_rank
    else:
        is_built_on_rank = ProcessGroupManager.is_tensor_parallel_first_rank()

    builder = BlendedMegatronDatasetBuilder(
        GPTDataset,
        sizes=list(_train_val_test_samples(args.training_parameters.num_training_steps, micro_batch_size, accumulation,
                                           args.training_parameters.eval_interval, class_args.get("eval_steps"))),
        config=GPTDatasetConfig(
            is_built_on_rank=is_built_on_rank,
            random_seed=class_args.get("seed", args.random_args.seed),
            sequence_length=sequence_length,
            blend=class_args.get("data_path"),
            blend_per_split=[class_args.get("train_data_path"), class_args.get("val_data_path"), class_args.get("test_data_path")],
            split=class_args.get("split"),
            path_to_cache=class_args.get("data_cache_path"),
            return_document_ids=False,
            fim_rate=class_args.get("fim_rate", 0),
            fim_spm_rate=class_args.get("fim_spm_rate", 0.5),
            node_uses_local_storage=class_args.get("node_uses_local_storage", False),
        ),
        tokenizer=tokenizer,
    )

    if class_args.get("data_path") is not None or class_args.get("train_data_path") is not None:
        train, val, test = builder.build()
        val, test = [val], [test]
    elif class_args.get("train_weighted_split_paths"):

        def groups_of(spec: list[dict] | None, which: Split) -> list:
            if spec is None:
                return []
            names, paths, ranges, weights = [], [], [], []
            for group in spec:
                assert len(group) == 1
                (name, members), = group.items()
                names.append([name] * len(members))
                paths.append([m["path"] for m in members])
                ranges.append([m["split"] for m in members])
                weights.append([m["weight"] for m in members])
            return builder.build_dataset_single_split(names, paths, ranges, weights, which)

        train_spec = class_args.get("train_weighted_split_paths")
        assert len(train_spec) == 1, "only 1 dataset group can be passed for training"
        train = groups_of(train_spec, Split.train)[0]
        val = groups_of(class_args.get("val_weighted_split_paths"), Split.valid)
        test = groups_of(class_args.get("test_weighted_split_paths"), Split.test)
    else:
        raise NotImplementedError("No dataloading argument passed")

    log_rank_0(logging.INFO, "> finished creating GPT datasets ...")

    def loader(dataset, consumed: int):
        if dispatching:
            missing = [dataset is None if is_built_on_rank else False]
            dist.broadcast_object_list(missing, src=source_rank, group=groups[source_rank])
            if missing[0]:
                return None
            sampler = None
            if is_built_on_rank:
                sampler = MegatronBatchSampler(total_samples=len(dataset), consumed_samples=consumed,
                                               micro_batch_size=samples_per_fetch * ranks_per_node, num_replicas=num_nodes, rank=node_rank)
            return iter(DispatchingDataLoader(dataset, batch_sampler=sampler, num_workers=num_workers, pin_memory=torch.cuda.is_available(),
                                              source_broadcast_mapping=groups, broadcast_world_size=ranks_per_node,
                                              static_shape_per_rank=(samples_per_fetch, sequence_length + 1), keys=["text"]))
        if dataset is None:
            return None
        sampler = MegatronBatchSampler(total_samples=len(dataset), consumed_samples=consumed, micro_batch_size=samples_per_fetch,
                                       num_replicas=ProcessGroupManager.get_data_parallel_world_size(),
                                       rank=ProcessGroupManager.get_data_parallel_rank())
        return iter(ResumableDataLoader(dataset, batch_sampler=sampler, num_workers=num_workers, pin_memory=torch.cuda.is_available()))

    return loader(train, consumed_samples), [loader(d, 0) for d in val], [loader(d, 0) for d in test]

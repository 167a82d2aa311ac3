"""The Megatron pretraining dataloaders on their own, for a training loop that is not this engine's (data parallelism only).

    python -m lm_engine.cli.megatron_dataloader --data-path 0.3 data/a_text 0.7 data/b_text --split 98,1,1 \
        --sequence-length 2048 --micro-batch-size 8 --num-training-steps 10000 --cache ./cache --show 2

    torchrun ... -m lm_engine.cli.megatron_dataloader ...      # every rank of a data-parallel job gets its own share

As a library: :func:`build_dataloaders` returns ``(train, validation list, test list)``; each batch is a dict with
``text`` of shape ``[micro_batch_size, sequence_length + 1]`` (the loss shifts by one token outside the loader).
Counterpart of the reference's example script tools/data/megatron_dataloader.py.
"""

from __future__ import annotations

from argparse import ArgumentParser
from contextlib import ExitStack

from ..arguments import DatasetArgs, DistributedArgs, RandomArgs, TrainingParameters
from ..utils import ProcessGroupManager


def _blend(values: list[str]) -> list:
    """``["0.3", "a", "0.7", "b"] -> [0.3, "a", 0.7, "b"]``; a list of plain paths stays one."""
    out = []
    for value in values:
        try:
            out.append(float(value))
        except ValueError:
            out.append(value)
    return out


def build_dataloaders(data_path: list, split: str, sequence_length: int, micro_batch_size: int, num_training_steps: int,
                      data_cache_path: str, tokenizer=None, seed: int = 42, gradient_accumulation_steps: int = 1,
                      eval_during_training: bool = False, eval_interval: int | None = None, eval_steps: int = 2,
                      consumed_samples: int = 0, fim_rate: float = 0.0, num_workers: int = 2):
    """Every rank of the (already initialised, or absent) process group is one data-parallel rank: the model-parallel
    view of the process-group manager is overridden for the duration of the construction. ``consumed_samples`` resumes
    in the middle of the data: ``global_step * micro_batch_size * gradient_accumulation_steps * world size``. The tokenizer
    is only needed for fill-in-the-middle (``fim_rate > 0``)."""
    from ..data.megatron import get_megatron_gpt_dataloaders

    class Arguments:
        random_args = RandomArgs(seed=seed)
        datasets = [DatasetArgs(class_name="MegatronDataset", data_name="Megatron", data_sampling_ratio=1, class_args={
            "eval_steps": eval_steps, "data_cache_path": data_cache_path, "data_path": data_path, "split": split,
            "sequence_length": sequence_length, "fim_rate": fim_rate, "num_workers": num_workers})]
        training_parameters = TrainingParameters(num_training_steps=num_training_steps, micro_batch_size=micro_batch_size,
                                                 gradient_accumulation_steps=gradient_accumulation_steps,
                                                 eval_interval=eval_interval, eval_during_training=eval_during_training)
        distributed_args = DistributedArgs()

    rank, world = ProcessGroupManager.get_global_rank(), ProcessGroupManager.get_world_size()
    with ExitStack() as stack:
        for manager in (ProcessGroupManager.set_dummy_data_parallel_world_size(world), ProcessGroupManager.set_dummy_data_parallel_rank(rank),
                        ProcessGroupManager.set_dummy_tensor_parallel_world_size(1), ProcessGroupManager.set_dummy_tensor_parallel_rank(0),
                        ProcessGroupManager.set_dummy_tensor_parallel_first_rank(rank)):
            stack.enter_context(manager)
        train, validation, test = get_megatron_gpt_dataloaders(Arguments(), tokenizer, consumed_samples=consumed_samples)
    return train, [loader for loader in validation if loader is not None], [loader for loader in test if loader is not None]


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--data-path", nargs="+", required=True, help="path prefixes, optionally each preceded by its weight")
    parser.add_argument("--split", default="100,0,0")
    parser.add_argument("--sequence-length", type=int, required=True)
    parser.add_argument("--micro-batch-size", type=int, required=True)
    parser.add_argument("--num-training-steps", type=int, required=True)
    parser.add_argument("--gradient-accumulation-steps", type=int, default=1)
    parser.add_argument("--cache", required=True, help="directory for the index caches")
    parser.add_argument("--seed", type=int, default=42)
    parser.add_argument("--consumed-samples", type=int, default=0)
    parser.add_argument("--tokenizer", default=None, help="only needed with --fim-rate")
    parser.add_argument("--fim-rate", type=float, default=0.0)
    parser.add_argument("--num-workers", type=int, default=0)
    parser.add_argument("--show", type=int, default=1, help="print this many training batches")
    args = parser.parse_args()

    tokenizer = None
    if args.tokenizer is not None:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(args.tokenizer)
    train, validation, test = build_dataloaders(
        _blend(args.data_path), args.split, args.sequence_length, args.micro_batch_size, args.num_training_steps, args.cache,
        tokenizer=tokenizer, seed=args.seed, gradient_accumulation_steps=args.gradient_accumulation_steps,
        consumed_samples=args.consumed_samples, fim_rate=args.fim_rate, num_workers=args.num_workers)
    print(f"rank {ProcessGroupManager.get_global_rank()} of {ProcessGroupManager.get_world_size()}: "
          f"{len(validation)} validation and {len(test)} test loaders")
    for index, batch in zip(range(args.show), train):
        text = batch["text"]
        print(f"batch {index}: text {tuple(text.shape)} {text.dtype}, first tokens {text[0, :8].tolist()}")


if __name__ == "__main__":
    main()

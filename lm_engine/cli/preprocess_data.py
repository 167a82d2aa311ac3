"""Tokenise text files (jsonl, jsonl.zst, arrow, or a dataset that ``datasets`` can stream) into Megatron ``.bin/.idx``
stores, optionally many inputs at once, and merge stores.

    python -m lm_engine.cli.preprocess_data convert --tokenizer T --input a.jsonl b.jsonl --output-prefix out/data
    python -m lm_engine.cli.preprocess_data merge --input out/data_0_text out/data_1_text --output-prefix out/all_text
    python -m lm_engine.cli.preprocess_data inspect --path-prefix out/all_text

Whole corpora laid out as ``<input-path>/<subset>/*.arrow`` (or ``*.jsonl`` / ``*.jsonl.zst``), the counterpart of the reference's
tools/data/convert_fms_data_to_megatron.py:

    python -m lm_engine.cli.preprocess_data convert-tree --tokenizer T --input-path raw --output-path tmp --data-subsets cc wiki \
        --jobs 16 --job-index $SLURM_ARRAY_TASK_ID           # one share of the files per job; finished files are skipped
    python -m lm_engine.cli.preprocess_data merge-tree --input-path tmp --output-path megatron --data-subsets cc wiki --max-file-size 100
"""

import json
import os
from argparse import ArgumentParser

from ..data.megatron.indexed_dataset import MMapIndexedDataset
from ..data.megatron.merge_data import merge_files
from ..data.megatron.preprocess_data import convert_file


_SOURCE_SUFFIXES = (".arrow", ".jsonl", ".jsonl.zst")


def source_files(input_path: str, subset: str) -> list[str]:
    """The convertible files of one subset directory, sorted by name."""
    return sorted(name for name in os.listdir(os.path.join(input_path, subset)) if name.endswith(_SOURCE_SUFFIXES))


def share_of_job(items: list, jobs: int, job_index: int) -> list:
    """Contiguous share ``job_index`` of ``jobs`` (sizes differ by at most one)."""
    assert 0 <= job_index < jobs, f"job index {job_index} outside 0..{jobs - 1}"
    return items[len(items) * job_index // jobs : len(items) * (job_index + 1) // jobs]


def convert_tree(tokenizer, input_path: str, output_path: str, subsets: list[str], jobs: int = 1, job_index: int = 0,
                 start_index: int | None = None, end_index: int | None = None, workers: int = 1, chunk_size: int = 1000,
                 json_keys: tuple[str, ...] = ("text",)) -> list[str]:
    """Converts this job's share of ``<input_path>/<subset>/*`` into ``<output_path>/<subset>/<file stem>_<key>.{bin,idx}`` and
    returns the prefixes written. A file whose index already exists is skipped, so an interrupted job can be repeated."""
    written = []
    for subset in subsets:
        names = share_of_job(source_files(input_path, subset)[start_index:end_index], jobs, job_index)
        os.makedirs(os.path.join(output_path, subset), exist_ok=True)
        for name in names:
            prefix = os.path.join(output_path, subset, name.split(".")[0])
            if all(os.path.isfile(f"{prefix}_{key}.idx") for key in json_keys):
                continue
            convert_file(tokenizer, os.path.join(input_path, subset, name), prefix, workers=workers, chunk_size=chunk_size,
                         json_keys=list(json_keys))
            written.append(prefix)
    return written


def groups_by_size(folder: str, max_size_gb: float | None) -> list[list[str]]:
    """Store prefixes of ``folder`` in name order, cut into groups whose ``.bin`` files add up to about ``max_size_gb``
    (a group is closed by the file that takes it over the limit); one group when there is no limit."""
    prefixes = sorted(os.path.join(folder, name[: -len(".bin")]) for name in os.listdir(folder) if name.endswith(".bin"))
    if max_size_gb is None:
        return [prefixes] if prefixes else []
    groups, current, size = [], [], 0
    for prefix in prefixes:
        current.append(prefix)
        size += os.path.getsize(prefix + ".bin")
        if size > max_size_gb * 1024**3:
            groups.append(current)
            current, size = [], 0
    if current:
        groups.append(current)
    return groups


def merge_tree(input_path: str, output_path: str, subsets: list[str], max_file_size: float | None = None,
               output_suffix: str | None = None) -> dict[str, list[str]]:
    """Merges the stores of every ``<input_path>/<subset>`` into ``<output_path>/<subset>[-<group>][-<suffix>]`` and records
    which inputs went into which output in ``<output_path>/files[-<suffix>].json``."""
    os.makedirs(output_path, exist_ok=True)
    suffix = f"-{output_suffix}" if output_suffix else ""
    made: dict[str, list[str]] = {}
    for subset in subsets:
        groups = groups_by_size(os.path.join(input_path, subset), max_file_size)
        for index, group in enumerate(groups):
            name = subset + (f"-{index}" if max_file_size is not None else "") + suffix
            merge_files(group, os.path.join(output_path, name))
            made[name] = group
    with open(os.path.join(output_path, f"files{suffix}.json"), "w") as handle:
        json.dump(made, handle, indent=4)
    return made


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    sub = parser.add_subparsers(dest="command", required=True)
    convert = sub.add_parser("convert")
    convert.add_argument("--tokenizer", required=True)
    convert.add_argument("--input", nargs="+", required=True)
    convert.add_argument("--output-prefix", required=True)
    convert.add_argument("--json-keys", nargs="+", default=["text"])
    convert.add_argument("--workers", type=int, default=1)
    convert.add_argument("--chunk-size", type=int, default=32)
    convert.add_argument("--subset", default=None)
    convert.add_argument("--no-append-eos", action="store_true")
    merge = sub.add_parser("merge")
    merge.add_argument("--input", nargs="+", required=True, help="path prefixes (without .bin / .idx)")
    merge.add_argument("--output-prefix", required=True)
    tree = sub.add_parser("convert-tree")
    tree.add_argument("--tokenizer", required=True)
    tree.add_argument("--input-path", required=True)
    tree.add_argument("--output-path", required=True)
    tree.add_argument("--data-subsets", nargs="+", required=True)
    tree.add_argument("--jobs", type=int, default=1, help="number of jobs the files are divided among")
    tree.add_argument("--job-index", type=int, default=0, help="which share this process converts (e.g. $SLURM_ARRAY_TASK_ID)")
    tree.add_argument("--start-index", type=int, default=None)
    tree.add_argument("--end-index", type=int, default=None)
    tree.add_argument("--workers", type=int, default=1)
    tree.add_argument("--json-keys", nargs="+", default=["text"])
    merge_all = sub.add_parser("merge-tree")
    merge_all.add_argument("--input-path", required=True)
    merge_all.add_argument("--output-path", required=True)
    merge_all.add_argument("--data-subsets", nargs="+", required=True)
    merge_all.add_argument("--max-file-size", type=float, default=None, help="size of a merged store in GB")
    merge_all.add_argument("--output-suffix", default=None)
    inspect = sub.add_parser("inspect")
    inspect.add_argument("--path-prefix", required=True)
    inspect.add_argument("--show", type=int, default=0, help="print the first N sequences")
    args = parser.parse_args()

    if args.command == "convert":
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(args.tokenizer)
        for index, path in enumerate(args.input):
            prefix = args.output_prefix if len(args.input) == 1 else f"{args.output_prefix}_{index}"
            convert_file(tokenizer, path, prefix, workers=args.workers, chunk_size=args.chunk_size, subset=args.subset,
                         json_keys=args.json_keys, append_eos_token=not args.no_append_eos)
    elif args.command == "merge":
        merge_files(args.input, args.output_prefix)
    elif args.command == "convert-tree":
        from transformers import AutoTokenizer

        written = convert_tree(AutoTokenizer.from_pretrained(args.tokenizer), args.input_path, args.output_path, args.data_subsets,
                               jobs=args.jobs, job_index=args.job_index, start_index=args.start_index, end_index=args.end_index,
                               workers=args.workers, json_keys=tuple(args.json_keys))
        print(f"job {args.job_index} of {args.jobs}: {len(written)} files converted")
    elif args.command == "merge-tree":
        for name, group in merge_tree(args.input_path, args.output_path, args.data_subsets, args.max_file_size, args.output_suffix).items():
            print(f"{name}: {len(group)} stores")
    else:
        store = MMapIndexedDataset(args.path_prefix)
        lengths = store.sequence_lengths
        print(f"sequences: {len(store)}  documents: {len(store.document_indices) - 1}  tokens: {int(lengths.sum())}  dtype: {store.index.dtype.__name__}")
        for i in range(min(args.show, len(store))):
            print(i, store[i].tolist())


if __name__ == "__main__":
    main()

"""Tokenise text files (jsonl, jsonl.zst, arrow, or a dataset that ``datasets`` can stream) into Megatron ``.bin/.idx``
stores, optionally many inputs at once, and merge stores.

    python -m lm_engine.cli.preprocess_data convert --tokenizer T --input a.jsonl b.jsonl --output-prefix out/data
    python -m lm_engine.cli.preprocess_data merge --input out/data_0_text out/data_1_text --output-prefix out/all_text
    python -m lm_engine.cli.preprocess_data inspect --path-prefix out/all_text
"""

from argparse import ArgumentParser

from ..data.megatron.indexed_dataset import MMapIndexedDataset
from ..data.megatron.merge_data import merge_files
from ..data.megatron.preprocess_data import convert_file


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
    else:
        store = MMapIndexedDataset(args.path_prefix)
        lengths = store.sequence_lengths
        print(f"sequences: {len(store)}  documents: {len(store.document_indices) - 1}  tokens: {int(lengths.sum())}  dtype: {store.index.dtype.__name__}")
        for i in range(min(args.show, len(store))):
            print(i, store[i].tolist())


if __name__ == "__main__":
    main()

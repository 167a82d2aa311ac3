"""Tokenise raw text into ``.bin``/``.idx`` stores, one per JSON key.

Parity: lm_engine/data/megatron/preprocess_data.py:21-111. Inputs: ``.jsonl``, ``.jsonl.zst`` (when ``zstandard`` is
installed), ``.arrow`` files of pre-tokenised documents (column ``tokens``), or anything ``datasets.load_dataset``
streams. Tokenisation runs in a process pool; the writer is the calling process.
"""

from __future__ import annotations

import io
import json
import multiprocessing

import numpy as np

from .indexed_dataset import DType, MMapIndexedDatasetBuilder


class ArrowIterator:
    def __init__(self, filename: str) -> None:
        import pyarrow as pa

        self.reader = pa.ipc.open_file(filename)
        self.num_records = self.reader.num_record_batches

    def __iter__(self):
        for i in range(self.num_records):
            yield self.reader.get_batch(i)["tokens"].to_numpy().tolist()


class Encoder:
    def __init__(self, tokenizer, json_keys: list[str], append_eod: bool) -> None:
        if isinstance(tokenizer, str):
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(tokenizer)
        self.tokenizer = tokenizer
        self.json_keys = json_keys
        self.append_eod = append_eod

    def _encode_data(self, data: dict) -> dict[str, list[int]]:
        out = {}
        for key in self.json_keys:
            ids = list(self.tokenizer.encode(data[key]))
            if ids:
                if self.append_eod:
                    ids.append(self.tokenizer.eos_token_id)
                out[key] = ids
        return out

    def encode(self, json_line: str) -> dict[str, list[int]]:
        return self._encode_data(json.loads(json_line))

    def encode_jsonl_zstd(self, raw: bytes) -> dict[str, list[int]]:
        return self.encode(raw.decode("utf-8"))

    def encode_hf(self, sample: dict) -> dict[str, list[int]]:
        return self._encode_data(sample)

    def convert_fms_arrow_to_megatron(self, tokens: list[int]) -> dict[str, list[int]]:
        if tokens and self.append_eod:
            tokens.append(self.tokenizer.eos_token_id)
        return {"text": tokens}


def _mapper(workers: int):
    if workers <= 1:
        return None, lambda fn, it, chunk: map(fn, it)
    pool = multiprocessing.Pool(workers)
    return pool, pool.imap


def convert_file(tokenizer, input_file: str, output_prefix: str, workers: int = 1, chunk_size: int = 32, subset: str | None = None,
                 json_keys: list[str] = ("text",), append_eos_token: bool = True) -> None:
    json_keys = list(json_keys)
    encoder = Encoder(tokenizer, json_keys, append_eos_token)
    pool, imap = _mapper(workers)
    handle = None
    try:
        if input_file.endswith(".jsonl"):
            assert subset is None, "jsonl doesn't support a subset"
            handle = open(input_file, "r", encoding="utf-8")
            encoded = imap(encoder.encode, handle, chunk_size)
        elif input_file.endswith(".jsonl.zst"):
            assert subset is None, "zst jsonl doesn't support a subset"
            from zstandard import ZstdDecompressor

            with open(input_file, "rb") as compressed:
                handle = io.BytesIO(ZstdDecompressor().stream_reader(compressed).read())
            encoded = imap(encoder.encode_jsonl_zstd, handle, chunk_size)
        elif input_file.endswith(".arrow"):
            assert subset is None, "arrow doesn't support a subset"
            encoded = imap(encoder.convert_fms_arrow_to_megatron, ArrowIterator(input_file), chunk_size)
        else:
            from datasets import load_dataset

            encoded = imap(encoder.encode_hf, load_dataset(input_file, streaming=True, split="train", data_dir=subset), chunk_size)

        dtype = DType.optimal_dtype(encoder.tokenizer.vocab_size)
        builders = {key: MMapIndexedDatasetBuilder(f"{output_prefix}_{key}.bin", dtype=dtype) for key in json_keys}
        for item in encoded:
            for key, document in item.items():
                builders[key].add_item(np.asarray(document, dtype=np.int64))
                builders[key].end_document()
        for key in json_keys:
            builders[key].finalize(f"{output_prefix}_{key}.idx")
    finally:
        if handle is not None:
            handle.close()
        if pool is not None:
            pool.close()
            pool.join()

"""Datasets read through the ``datasets`` library (parity: lm_engine/data/huggingface.py)."""

from __future__ import annotations

from ..enums import DatasetSplit, Mode
from .base import BaseDataset


class HuggingFaceDataset(BaseDataset):
    """``class_args``: ``data_path`` (hub name or local path), ``input_key``, ``output_key`` and optional
    ``data_files`` / ``name``; the split follows the datasets-library naming (``train`` / ``validation`` / ``test``)."""

    _SPLIT_NAME = {DatasetSplit.train: "train", DatasetSplit.val: "validation", DatasetSplit.test: "test"}

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.examples = self.prepare_examples()

    def prepare_examples(self) -> list[dict]:
        from datasets import load_dataset

        ca = self.class_args
        split = self._SPLIT_NAME[self.split]
        dataset = load_dataset(ca["data_path"], name=ca.get("name"), data_files=ca.get("data_files"), split=None)
        if split not in dataset:
            return []
        input_key = ca.get("input_key", "input")
        output_key = ca.get("output_key", "output")
        examples = []
        for raw in dataset[split]:
            text_in = self.construct_input_from_format(raw[input_key])
            text_out = self.construct_output_from_format(raw[output_key]) if self.mode == Mode.training else None
            examples.append(self.get_input_output_token_ids(text_in, text_out))
        return examples

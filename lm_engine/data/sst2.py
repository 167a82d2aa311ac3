"""GLUE SST-2 sentiment classification cast as text generation (parity: lm_engine/data/sst2.py)."""

from __future__ import annotations

from ..enums import DatasetSplit, Mode
from .base import BaseDataset


class SST2Dataset(BaseDataset):
    _SPLIT_NAME = {DatasetSplit.train: "train", DatasetSplit.val: "validation", DatasetSplit.test: "test"}

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        from datasets import load_dataset

        data = load_dataset("glue", "sst2")[self._SPLIT_NAME[self.split]]
        for raw in data:
            text_in = self.construct_input_from_format(raw["sentence"].strip())
            # the label as a word, as in the reference (lm_engine/data/sst2.py:53-57)
            text_out = (self.construct_output_from_format("positive" if raw["label"] == 1 else "negative")
                        if self.mode == Mode.training else None)
            self.examples.append(self.get_input_output_token_ids(text_in, text_out))

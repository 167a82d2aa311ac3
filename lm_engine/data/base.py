"""Finetuning dataset base classes (parity: lm_engine/data/base.py:12-200).

An example is ``{"input": ids, "output": ids}``: for decoder-only models ``input`` already holds prompt + answer +
EOS and ``output`` the answer + EOS (the loss mask is derived from the length difference); for encoder-decoder
models ``input`` is the prompt + EOS. Prompts are built by substituting the raw text for ``__input__`` /
``__output__`` in the configured formats.
"""

from __future__ import annotations

import torch

from ..defaults import INPUT_FORMAT, OUTPUT_FORMAT
from ..enums import DatasetSplit, Mode


class BaseDataset(torch.utils.data.Dataset):
    def __init__(self, class_args: dict, split: DatasetSplit, mode: Mode, tokenizer, is_encoder_decoder: bool,
                 data_name: str, input_format: str, output_format: str, max_input_tokens: int | None,
                 max_output_tokens: int | None) -> None:
        super().__init__()
        self.class_args = class_args
        self.split = split
        self.mode = mode
        self.tokenizer = tokenizer
        self.is_encoder_decoder = is_encoder_decoder
        self.data_name = data_name
        self.input_format = input_format
        self.output_format = output_format
        # budgets exclude the EOS token that is appended
        self.max_input_tokens = None if max_input_tokens is None else max_input_tokens - (1 if is_encoder_decoder else 0)
        self.max_output_tokens = None if max_output_tokens is None else max_output_tokens - 1
        self.examples: list[dict] = []

    def construct_input_from_format(self, text: str) -> str:
        return text if self.input_format == INPUT_FORMAT else self.input_format.replace(INPUT_FORMAT, text, 1)

    def construct_output_from_format(self, text: str) -> str:
        return text if self.output_format == OUTPUT_FORMAT else self.output_format.replace(OUTPUT_FORMAT, text, 1)

    def get_input_output_token_ids(self, input: str, output: str | None) -> dict:
        eos = self.tokenizer.eos_token_id
        prompt = list(self.tokenizer(input, add_special_tokens=False)["input_ids"])
        if self.is_encoder_decoder:
            if self.max_input_tokens is not None:
                prompt = prompt[: self.max_input_tokens - 1]
            prompt.append(eos)
        elif self.max_input_tokens is not None:
            prompt = prompt[: self.max_input_tokens]
        if self.mode != Mode.training:
            return {"input": prompt}
        answer = list(self.tokenizer(output, add_special_tokens=False)["input_ids"])
        if self.max_output_tokens is not None:
            answer = answer[: self.max_output_tokens - 1]
        answer.append(eos)
        if not self.is_encoder_decoder:
            prompt = prompt + answer
        return {"input": prompt, "output": answer}

    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, state_dict: dict) -> None:
        return None

    def __getitem__(self, index: int) -> dict:
        return self.examples[index]

    def __len__(self) -> int:
        return len(self.examples)


class BlendedDatasets(torch.utils.data.Dataset):
    """Concatenation of datasets with a ``global index -> (dataset, local index)`` map."""

    def __init__(self, datasets: list[BaseDataset], split: DatasetSplit) -> None:
        super().__init__()
        self.split = split
        self.datasets = datasets
        self.num_examples = sum(self.get_num_examples_in_each_dataset())
        self.indexing_array: list[tuple[int, int]] = []
        for d, dataset in enumerate(datasets):
            self.indexing_array.extend((d, i) for i in range(len(dataset)))

    def get_num_datasets(self) -> int:
        return len(self.datasets)

    def get_num_examples_in_each_dataset(self) -> list[int]:
        return [len(d) for d in self.datasets]

    def state_dict(self) -> dict:
        return {d.data_name: d.state_dict() for d in self.datasets}

    def load_state_dict(self, state_dict: dict) -> None:
        for d in self.datasets:
            d.load_state_dict(state_dict.get(d.data_name, {}))

    def __len__(self) -> int:
        return self.num_examples

    def __getitem__(self, index: int) -> dict:
        d, i = self.indexing_array[index]
        return self.datasets[d][i]

    def __repr__(self) -> str:
        lines = [f"number of datasets = {self.get_num_datasets()}", f"total examples in the entire dataset mixture = {len(self)}"]
        for dataset in self.datasets:
            lines.append(f"examples in {type(dataset).__name__} ({dataset.data_name}) = {len(dataset)}")
        return "\n".join(lines)

"""Synthetic finetuning dataset of constant-token examples for profiling and timing (parity: lm_engine/data/debug.py)."""

from __future__ import annotations

from ..defaults import INPUT_FORMAT, OUTPUT_FORMAT
from ..enums import Mode
from .base import BaseDataset


class DebugDataset(BaseDataset):
    """``class_args``: ``num_examples``; ``token_id`` (default: the end-of-sequence token); ``static_examples`` (default true:
    every example is the same; false: example ``i`` is made of token ``i``). As in the reference an example is not put
    together from a prompt and an answer: ``input`` holds ``max_input_tokens`` tokens, which is then the sequence length
    of the batch, and ``output`` (training only) ``max_output_tokens`` tokens, the labels of the last positions."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        if self.input_format != INPUT_FORMAT or self.output_format != OUTPUT_FORMAT:
            raise ValueError("input_format and output_format are not used by the debug dataset")
        self._length = self.class_args.get("num_examples")
        assert isinstance(self._length, int) and self._length > 0, "class_args.num_examples must be a positive integer"
        self._token_id = self.class_args.get("token_id", self.tokenizer.eos_token_id if self.tokenizer is not None else 0)
        self._static_examples = self.class_args.get("static_examples", True)
        self._example = self._make(self._token_id) if self._static_examples else None

    def _make(self, token_id: int) -> dict:
        prompt = [token_id] * (self.max_input_tokens if self.max_input_tokens is not None else 8)
        if self.mode != Mode.training:
            return {"input": prompt}
        # `max_output_tokens` was reduced by one on construction to leave room for the end-of-sequence token
        return {"input": prompt, "output": [token_id] * (self.max_output_tokens + 1 if self.max_output_tokens is not None else 8)}

    def __getitem__(self, index: int) -> dict:
        example = self._example if self._static_examples else self._make(index)
        return {key: list(value) for key, value in example.items()}

    def __len__(self) -> int:
        return self._length

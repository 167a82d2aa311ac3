"""Synthetic finetuning dataset of constant-token examples (parity: lm_engine/data/debug.py)."""

from __future__ import annotations

from .base import BaseDataset


class DebugDataset(BaseDataset):
    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        if self.do_format():
            raise ValueError("input_format and output_format are not used by the debug dataset")
        self._length = self.class_args.get("num_examples")
        token = self.class_args.get("token_id", self.tokenizer.eos_token_id if self.tokenizer is not None else 0)
        answer = [token] * (self.max_output_tokens + 1 if self.max_output_tokens is not None else 8)
        prompt = [token] * (self.max_input_tokens if self.max_input_tokens is not None else 8)
        if self.is_encoder_decoder:
            self._example = {"input": prompt, "output": answer}
        else:
            self._example = {"input": prompt + answer, "output": answer}

    def do_format(self) -> bool:
        from ..defaults import INPUT_FORMAT, OUTPUT_FORMAT

        return self.input_format != INPUT_FORMAT or self.output_format != OUTPUT_FORMAT

    def __getitem__(self, index: int) -> dict:
        return {k: list(v) for k, v in self._example.items()}

    def __len__(self) -> int:
        return self._length

"""Instruction-tuning datasets (parity: lm_engine/data/instruction_tuning/{base,alpaca,dolly,slimorca}.py)."""

from __future__ import annotations

from ..enums import DatasetSplit, Mode
from .base import BaseDataset


class BaseInstructionDataset(BaseDataset):
    hub_name: str | None = None

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        if self.split != DatasetSplit.train:
            return  # these corpora only ship a train split
        self.examples = self.prepare_examples()

    def construct_input_from_format(self, instruction: str, input: str | None = None) -> str:
        """The prompt of the reference (lm_engine/data/instruction_tuning/base.py:43-48): the instruction, a blank line, an
        ``input:`` line when there is one, and ``output:``. The reference refuses an ``input_format`` for these datasets;
        here one wraps the whole prompt."""
        text = instruction + "\n\n"
        if input:
            text += f"input: {input}\n"
        text += "output:"
        return super().construct_input_from_format(text)

    def load_raw(self):
        from datasets import load_dataset

        return load_dataset(self.class_args.get("data_path", self.hub_name))["train"]

    def fields(self, raw: dict) -> tuple[str, str | None, str]:
        raise NotImplementedError

    def prepare_examples(self) -> list[dict]:
        examples = []
        for raw in self.load_raw():
            instruction, context, answer = self.fields(raw)
            text_in = self.construct_input_from_format(instruction, context)
            text_out = self.construct_output_from_format(answer.strip()) if self.mode == Mode.training else None
            examples.append(self.get_input_output_token_ids(text_in, text_out))
        return examples


class AlpacaDataset(BaseInstructionDataset):
    hub_name = "tatsu-lab/alpaca"

    def fields(self, raw):
        return raw["instruction"], raw.get("input"), raw["output"]


class DollyDataset(BaseInstructionDataset):
    hub_name = "databricks/databricks-dolly-15k"

    def fields(self, raw):
        return raw["instruction"], raw.get("context"), raw["response"]


class SlimOrcaDataset(BaseInstructionDataset):
    hub_name = "Open-Orca/SlimOrca-Dedup"

    def fields(self, raw):
        turns = raw["conversations"]
        if len(turns) == 3:  # system prompt (possibly empty), question, answer: the layout of the corpus
            return turns[0]["value"], turns[1]["value"], turns[2]["value"]
        said = {turn["from"]: turn["value"] for turn in turns}
        return said.get("system", ""), said.get("human"), said.get("gpt", "")

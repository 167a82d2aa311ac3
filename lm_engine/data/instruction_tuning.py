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
        text = instruction if not input else f"{instruction}\n\n{input}"
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
            text_out = self.construct_output_from_format(answer) if self.mode == Mode.training else None
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
        system = human = answer = ""
        for turn in raw["conversations"]:
            if turn["from"] == "system":
                system = turn["value"]
            elif turn["from"] == "human":
                human = turn["value"]
            elif turn["from"] == "gpt":
                answer = turn["value"]
        return (system if system else human), (human if system else None), answer

"""Batch collation for finetuning / inference (parity: lm_engine/data/utils.py:14-165)."""

from __future__ import annotations

import math

import torch

from ..enums import LossMask, Mode
from ..hf_models import convert_padding_free_lists_to_tensors


def collate_fn(batch: list[dict], mode: Mode, loss_mask: LossMask, eos_token_id: int, is_encoder_decoder: bool,
               use_padding_free_transformer: bool, labels_mask_value: int = -100, pad_to_multiple_of: int = 1,
               device: torch.device | None = None) -> dict:
    """Padding-free: one flat token stream with ``cu_seqlens`` / ``position_ids`` (prompt tokens masked with -100 for
    ``output_only``; the LAST document is right-padded so that the token count is a multiple of
    ``pad_to_multiple_of``). Padded: LEFT padding with EOS plus an attention mask."""
    inputs = [list(example["input"]) for example in batch]
    outputs = [list(example["output"]) for example in batch] if mode == Mode.training else None
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")

    def masked(array_in: list[int], array_out: list[int], width: int | None = None) -> list[int]:
        width = len(array_in) if width is None else width
        return [labels_mask_value] * (width - len(array_out)) + array_out

    if use_padding_free_transformer:
        if is_encoder_decoder:
            raise NotImplementedError("the padding-free transformer supports decoder-only models")
        labels = None
        if outputs is not None:
            if loss_mask == LossMask.output_only:
                labels = [masked(i, o) for i, o in zip(inputs, outputs)]
            elif loss_mask == LossMask.no_mask:
                labels = [list(i) for i in inputs]
            else:
                raise ValueError(f"unexpected loss_mask ({loss_mask})")
        if pad_to_multiple_of > 1:
            total = sum(len(i) for i in inputs)
            extra = math.ceil(total / pad_to_multiple_of) * pad_to_multiple_of - total
            inputs[-1].extend([eos_token_id] * extra)
            if labels is not None:
                labels[-1].extend([labels_mask_value] * extra)
        input_ids, position_ids, _, labels_t, cu_seqlens, max_seqlen = convert_padding_free_lists_to_tensors(
            input_ids=inputs, labels=labels, device=device)
        result = {"input_ids": input_ids, "position_ids": position_ids, "cu_seqlens": cu_seqlens, "max_seqlen": max_seqlen}
        if labels_t is not None:
            result["labels"] = labels_t
        return result

    labels = None
    if is_encoder_decoder:
        if pad_to_multiple_of > 1:
            raise NotImplementedError("pad_to_multiple_of is not implemented for encoder-decoder models")
        width = max(map(len, inputs))
        if outputs is not None:
            if loss_mask != LossMask.output_only:
                raise ValueError("only the output_only loss mask is supported with encoder-decoder models")
            out_width = max(map(len, outputs))
            labels = [o + [labels_mask_value] * (out_width - len(o)) for o in outputs]
    else:
        width = max(map(len, inputs))
        if pad_to_multiple_of > 1:
            width = math.ceil(width / pad_to_multiple_of) * pad_to_multiple_of
        if outputs is not None:
            if loss_mask == LossMask.output_only:
                labels = [masked(i, o, width) for i, o in zip(inputs, outputs)]
            elif loss_mask == LossMask.no_mask:
                labels = [[labels_mask_value] * (width - len(i)) + i for i in inputs]
            else:
                raise ValueError(f"unexpected loss_mask ({loss_mask})")
    input_ids = [[eos_token_id] * (width - len(i)) + i for i in inputs]
    attention_mask = [[0] * (width - len(i)) + [1] * len(i) for i in inputs]
    result = {"input_ids": torch.tensor(input_ids, device=device), "attention_mask": torch.tensor(attention_mask, device=device)}
    if labels is not None:
        result["labels"] = torch.tensor(labels, device=device)
    return result

"""Autoregressive decoding loop over the model's own generation cache (greedy, temperature, top-k, top-p)."""

from __future__ import annotations

from types import SimpleNamespace

import torch


def _filter_logits(logits: torch.Tensor, top_k: int | None, top_p: float | None) -> torch.Tensor:
    if top_k is not None and top_k > 0:
        kth = logits.topk(min(top_k, logits.shape[-1]), dim=-1).values[..., -1, None]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        sorted_logits, order = logits.sort(dim=-1, descending=True)
        cumulative = sorted_logits.softmax(-1).cumsum(-1)
        drop = cumulative - sorted_logits.softmax(-1) > top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)
    return logits


@torch.no_grad()
def decode(model, input_ids: torch.Tensor, attention_mask: torch.Tensor | None, max_new_tokens: int, do_sample: bool,
           temperature: float | None, top_k: int | None, top_p: float | None, eos_token_id: int | None,
           pad_token_id: int | None, return_dict: bool, output_scores: bool):
    device = input_ids.device
    batch = input_ids.shape[0]
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    sequences = input_ids
    finished = torch.zeros(batch, dtype=torch.bool, device=device)
    scores = []
    cache = None
    step_input = input_ids
    for _ in range(max_new_tokens):
        out = model(input_ids=step_input, attention_mask=attention_mask, past_key_values=cache, use_cache=True)
        cache = out.past_key_values
        logits = out.logits[:, -1, :].float()
        if output_scores:
            scores.append(logits)
        if do_sample:
            if temperature is not None and temperature > 0:
                logits = logits / temperature
            probs = _filter_logits(logits, top_k, top_p).softmax(-1)
            next_token = torch.multinomial(probs, 1).squeeze(-1)
        else:
            next_token = logits.argmax(-1)
        if eos_token_id is not None:
            fill = pad_token_id if pad_token_id is not None else eos_token_id
            next_token = torch.where(finished, torch.full_like(next_token, fill), next_token)
            finished = finished | (next_token == eos_token_id)
        sequences = torch.cat([sequences, next_token[:, None]], dim=1)
        attention_mask = torch.cat([attention_mask, attention_mask.new_ones(batch, 1)], dim=1)
        step_input = next_token[:, None]
        if eos_token_id is not None and bool(finished.all()):
            break
    if return_dict:
        return SimpleNamespace(sequences=sequences, scores=tuple(scores) if output_scores else None)
    return sequences

"""Input helpers (parity: lm_engine/hf_models/utils.py:10-82)."""

from __future__ import annotations

from contextlib import contextmanager

import torch

_GENERATION_CACHE_ENABLED = True


def convert_padding_free_lists_to_tensors(
    input_ids: list[list[int]] | None = None,
    inputs_embeds: list[list[float]] | None = None,
    position_ids: list[list[int]] | None = None,
    token_type_ids: list[list[int]] | None = None,
    labels: list[list[int]] | None = None,
    device: torch.device | None = None,
):
    """Flatten nested per-document lists into packed tensors plus ``cu_seqlens`` (int32) and ``max_seqlen``."""
    if inputs_embeds is not None:
        raise NotImplementedError("nested inputs_embeds are not supported with the padding-free transformer")
    lengths = [len(doc) for doc in input_ids]
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=device)
    max_seqlen = max(lengths)

    def flat(nested, dtype=torch.long):
        if nested is None:
            return None
        return torch.tensor([v for doc in nested for v in doc], dtype=dtype, device=device)

    if position_ids is None:
        position_ids = [list(range(n)) for n in lengths]
    return flat(input_ids), flat(position_ids), flat(token_type_ids), flat(labels), cu_seqlens, max_seqlen


@contextmanager
def disable_generation_cache():
    """Training never needs a KV cache; inside this context the models do not create one."""
    global _GENERATION_CACHE_ENABLED
    previous = _GENERATION_CACHE_ENABLED
    _GENERATION_CACHE_ENABLED = False
    try:
        yield
    finally:
        _GENERATION_CACHE_ENABLED = previous


def is_generation_cache_enabled() -> bool:
    return _GENERATION_CACHE_ENABLED

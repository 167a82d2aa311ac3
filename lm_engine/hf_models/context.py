"""Per-forward sequence bookkeeping shared by all layers of a model.

A batch is either *padded* (``[batch, seq]`` tensors plus an optional 0/1 ``attention_mask``) or *packed*
(padding-free: all tokens of all documents concatenated to ``[T]`` with ``cu_seqlens``/``max_seqlen`` and per-token
``position_ids``). Layers read what they need from this object instead of receiving half a dozen arguments.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class SequenceContext:
    packed: bool
    batch_size: int
    query_length: int
    key_length: int
    position_ids: torch.Tensor | None = None
    cu_seqlens: torch.Tensor | None = None
    max_seqlen: int | None = None
    attention_mask: torch.Tensor | None = None  # [batch, key_length] of 0/1 (padded mode only)
    rope_cos_sin: tuple[torch.Tensor, torch.Tensor] | None = None  # gathered per position, broadcastable to heads
    rope_half_tables: tuple[torch.Tensor, torch.Tensor] | None = None  # fp32 [max_pos, rope_dim/2]
    _bool_mask: torch.Tensor | None = field(default=None, repr=False)
    _pos_i32: torch.Tensor | None = field(default=None, repr=False)
    _cu_i32: torch.Tensor | None = field(default=None, repr=False)

    def position_ids_int32(self) -> torch.Tensor:
        if self._pos_i32 is None:
            self._pos_i32 = self.position_ids.to(torch.int32).contiguous()
        return self._pos_i32

    def cu_seqlens_int32(self) -> torch.Tensor:
        if self._cu_i32 is None:
            self._cu_i32 = self.cu_seqlens.to(torch.int32).contiguous()
        return self._cu_i32

    @property
    def past_length(self) -> int:
        return self.key_length - self.query_length

    def boolean_attention_mask(self, device) -> torch.Tensor | None:
        """``[batch, 1, query, key]`` mask (True = attend) combining causality and padding; None when the plain
        causal flag of the attention kernel is sufficient."""
        if self.packed:
            return None
        if self.attention_mask is None and self.past_length == 0:
            return None
        if self._bool_mask is None:
            q, k = self.query_length, self.key_length
            rows = torch.arange(self.past_length, k, device=device)[:, None]
            cols = torch.arange(k, device=device)[None, :]
            mask = (cols <= rows)[None, None].expand(self.batch_size, 1, q, k)
            if self.attention_mask is not None:
                mask = mask & self.attention_mask.to(device=device, dtype=torch.bool)[:, None, None, :]
            self._bool_mask = mask
        return self._bool_mask

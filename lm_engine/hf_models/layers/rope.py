"""Rotary position embedding in the half-rotation form, with partial rotation and YaRN scaling.

Parity: lm_engine/hf_models/modeling_utils/position_embedding/rope.py:13-161. The table is fp32
``[max_position, head_dim]`` (frequencies repeated over both halves) times ``mscale``; when ``rope_dim`` is smaller
than the head width only the LAST ``rope_dim`` channels rotate.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = torch.chunk(x, 2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(x: torch.Tensor, cos_sin: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    cos, sin = cos_sin
    rd = cos.shape[-1]
    if rd == x.shape[-1]:
        return (x * cos) + (rotate_half(x) * sin)
    keep, rot = x[..., :-rd], x[..., -rd:]
    rot = (rot * cos) + (rotate_half(rot) * sin)
    return torch.cat([keep, rot], dim=-1)


class RoPE(nn.Module):
    def __init__(self, head_dim: int, max_position_embeddings: int = 2048, base: int = 10000) -> None:
        super().__init__()
        self.head_dim = head_dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base
        self.mscale = 1.0
        self.reset_parameters()

    def _inverse_frequencies(self) -> torch.Tensor:
        return 1.0 / (self.base ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim))

    @torch.no_grad()
    def reset_parameters(self) -> None:
        self.register_buffer("inv_freq", self._inverse_frequencies(), persistent=False)
        self._build(self.max_position_embeddings)

    def _build(self, seq_len: int, device=None) -> None:
        self.max_seq_len_cached = seq_len
        inv = self.inv_freq if device is None else self.inv_freq.to(device)
        t = torch.arange(seq_len, dtype=torch.float32, device=inv.device)
        freqs = torch.outer(t, inv)
        self.register_buffer("cos_half", (freqs.cos() * self.mscale).contiguous(), persistent=False)
        self.register_buffer("sin_half", (freqs.sin() * self.mscale).contiguous(), persistent=False)

    def ensure(self, seq_len: int, device) -> None:
        if seq_len > self.max_seq_len_cached or self.cos_half.device != torch.device(device):
            self._build(max(seq_len, self.max_seq_len_cached), device=device)

    def half_tables(self, seq_len: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        """fp32 ``[seq_len, head_dim / 2]`` cos and sin tables (what the fused kernel consumes)."""
        self.ensure(seq_len, device)
        return self.cos_half, self.sin_half

    def forward(self, seq_len: int, dtype: torch.dtype, device=None) -> tuple[torch.Tensor, torch.Tensor]:
        device = self.cos_half.device if device is None else device
        self.ensure(seq_len, device)
        cos = torch.cat([self.cos_half[:seq_len], self.cos_half[:seq_len]], dim=-1).to(dtype)
        sin = torch.cat([self.sin_half[:seq_len], self.sin_half[:seq_len]], dim=-1).to(dtype)
        return cos, sin


class YaRNScaledRoPE(RoPE):
    """YaRN (arXiv 2309.00071): interpolate low frequencies, keep high ones, scale magnitudes by ``mscale``."""

    def __init__(self, head_dim: int, max_position_embeddings: int = 2048, base: int = 10000, scale: float = 1,
                 original_max_position_embeddings: int = 2048, extrapolation_factor: float = 1,
                 attn_factor: float = 1, beta_fast: int = 32, beta_slow: int = 1) -> None:
        nn.Module.__init__(self)
        self.head_dim = head_dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base
        self.scale = scale
        self.original_max_position_embeddings = original_max_position_embeddings
        self.extrapolation_factor = extrapolation_factor
        self.attn_factor = attn_factor
        self.beta_fast = beta_fast
        self.beta_slow = beta_slow
        self.mscale = (0.1 * math.log(scale) + 1.0 if scale > 1 else 1.0) * attn_factor
        self.reset_parameters()

    def _correction_dim(self, rotations: float) -> float:
        return (self.head_dim * math.log(self.original_max_position_embeddings / (rotations * 2 * math.pi))) / (
            2 * math.log(self.base)
        )

    def _inverse_frequencies(self) -> torch.Tensor:
        pos = self.base ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim)
        extrapolated = 1.0 / pos
        interpolated = 1.0 / (self.scale * pos)
        low = max(math.floor(self._correction_dim(self.beta_fast)), 0)
        high = min(math.ceil(self._correction_dim(self.beta_slow)), self.head_dim - 1)
        if low == high:
            high += 0.001
        ramp = torch.clamp((torch.arange(self.head_dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
        keep = (1 - ramp) * self.extrapolation_factor
        return interpolated * (1 - keep) + extrapolated * keep

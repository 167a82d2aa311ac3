"""Causal softmax attention over packed (padding-free) sequences.

Native path: tcgen05 forward/backward kernels that read q, k and v straight out of the fused projection buffer
(layout ``[T, groups, (q_per_group + 2), head_dim]``) through strided TMA maps, so no head split/copy is made.
Oracle / CPU path: per-document ``scaled_dot_product_attention`` in the input dtype.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import native, native_available, note_fallback, status_word
from .timeline import site


def split_fused_qkv(qkv: torch.Tensor, groups: int, qpg: int, d: int):
    """Views of q ``[T, groups*qpg, d]``, k and v ``[T, groups, d]`` inside a fused projection."""
    T = qkv.shape[0]
    v4 = qkv.view(T, groups, qpg + 2, d)
    q = v4[:, :, :qpg].reshape(T, groups * qpg, d)
    k = v4[:, :, qpg]
    v = v4[:, :, qpg + 1]
    return q, k, v


def attention_varlen_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                               scale: float | None, causal: bool = True, dropout_p: float = 0.0,
                               sliding_window: int | None = None, softcap: float = 0.0) -> torch.Tensor:
    """q ``[T, hq, d]``, k/v ``[T, hkv, d]`` -> ``[T, hq, d]``; documents delimited by ``cu_seqlens``.

    ``sliding_window`` (a query sees the keys at most that many positions before it, and after it when not causal) and
    ``softcap`` (scores become ``softcap * tanh(scores / softcap)``) follow the flash-attention meaning of the reference's
    helper (lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/flash_attention_utils.py:65-81); they are evaluated
    with explicit score matrices."""
    if sliding_window is not None or softcap:
        return _attention_varlen_windowed(q, k, v, cu_seqlens, scale, causal, dropout_p, sliding_window, softcap)
    bounds = cu_seqlens.tolist()
    outs = []
    hq, hkv = q.shape[1], k.shape[1]
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e == s:
            continue
        qi = q[s:e].transpose(0, 1).unsqueeze(0)
        ki = k[s:e].transpose(0, 1).unsqueeze(0)
        vi = v[s:e].transpose(0, 1).unsqueeze(0)
        if hq != hkv:
            ki = ki.repeat_interleave(hq // hkv, dim=1)
            vi = vi.repeat_interleave(hq // hkv, dim=1)
        o = F.scaled_dot_product_attention(qi, ki, vi, is_causal=causal, scale=scale, dropout_p=dropout_p)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, dim=0)


def _attention_varlen_windowed(q, k, v, cu_seqlens, scale, causal, dropout_p, sliding_window, softcap) -> torch.Tensor:
    bounds = cu_seqlens.tolist()
    outs = []
    hq, hkv, d = q.shape[1], k.shape[1], q.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e == s:
            continue
        n = e - s
        qi, ki, vi = q[s:e].transpose(0, 1).float(), k[s:e].transpose(0, 1).float(), v[s:e].transpose(0, 1).float()
        if hq != hkv:
            ki, vi = ki.repeat_interleave(hq // hkv, dim=0), vi.repeat_interleave(hq // hkv, dim=0)
        scores = torch.einsum("hqd,hkd->hqk", qi, ki) * scale
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        i = torch.arange(n, device=q.device)[:, None]
        j = torch.arange(n, device=q.device)[None, :]
        allowed = (j <= i) if causal else torch.ones(n, n, dtype=torch.bool, device=q.device)
        if sliding_window is not None:
            allowed = allowed & (j >= i - sliding_window) & (j <= i + sliding_window)
        probs = torch.softmax(scores.masked_fill(~allowed, float("-inf")), dim=-1)
        if dropout_p:
            probs = F.dropout(probs, dropout_p)
        outs.append(torch.einsum("hqk,hkd->hqd", probs, vi).transpose(0, 1).to(q.dtype))
    return torch.cat(outs, dim=0)


def _native_attention_ok(qkv: torch.Tensor, d: int) -> bool:
    if not (native_available() and qkv.is_cuda and qkv.dtype == torch.bfloat16):
        return False
    return hasattr(native(), "attn_fwd") and d in (64, 128) and qkv.stride(-1) == 1 and qkv.stride(0) % 8 == 0


class _FusedQKVAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cu_seqlens, max_seqlen, groups, qpg, d, scale, causal):
        C = native()
        with site("attention.fwd"):
            out, lse = C.attn_fwd(qkv, cu_seqlens, int(max_seqlen), groups, qpg, d, float(scale), causal, status_word(qkv.device))
        ctx.save_for_backward(qkv, out, lse, cu_seqlens)
        ctx.meta = (int(max_seqlen), groups, qpg, d, float(scale), causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, cu_seqlens = ctx.saved_tensors
        max_seqlen, groups, qpg, d, scale, causal = ctx.meta
        with site("attention.bwd"):
            dqkv = native().attn_bwd(dout.contiguous(), qkv, out, lse, cu_seqlens, max_seqlen, groups, qpg, d, scale, causal, status_word(qkv.device))
        return dqkv, None, None, None, None, None, None, None


def padded_head_dim(d: int) -> int | None:
    """The head width the kernels run for a head of width ``d``: 64 or 128 themselves, the next of the two for any
    other multiple of 8 up to 128 (80 and 96 run as 128, 32 as 64), ``None`` when the kernels cannot take it."""
    if d in (64, 128):
        return d
    if d % 8 or d > 128 or d <= 0:
        return None
    return 64 if d < 64 else 128


def pad_fused_qkv(qkv: torch.Tensor, groups: int, qpg: int, d: int, dp: int) -> torch.Tensor:
    """``[T, groups * (qpg + 2) * d] -> [T, groups * (qpg + 2) * dp]`` with every head zero-padded to ``dp`` channels.
    Zero key / query channels add nothing to the scores and zero value channels give zero output channels, so attention
    over the padded heads, cut back to ``d`` channels, is attention over the original heads (differentiable)."""
    T = qkv.shape[0]
    return F.pad(qkv.view(T, groups * (qpg + 2), d), (0, dp - d)).view(T, groups * (qpg + 2) * dp)


def attention_fused_qkv(qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int, groups: int, qpg: int, d: int,
                        scale: float | None = None, causal: bool = True, dropout_p: float = 0.0,
                        sliding_window: int | None = None, softcap: float = 0.0) -> torch.Tensor:
    """Attention over a fused projection ``[T, groups*(qpg+2)*d]`` -> ``[T, groups*qpg*d]``.

    A sliding window or a score cap is not in the kernels: such a call is counted as a fallback (an error in strict mode)
    and evaluated by the PyTorch formulation."""
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if sliding_window is not None or softcap:
        note_fallback("attention", "sliding window / score cap", qkv)
        q, k, v = split_fused_qkv(qkv, groups, qpg, d)
        out = attention_varlen_reference(q, k, v, cu_seqlens, scale, causal, dropout_p, sliding_window, softcap)
        return out.reshape(qkv.shape[0], groups * qpg * d)
    if dropout_p == 0.0 and _native_attention_ok(qkv, d):
        return _FusedQKVAttentionFn.apply(qkv, cu_seqlens.to(torch.int32), max_seqlen, groups, qpg, d, scale, causal)
    dp = padded_head_dim(d)
    if dropout_p == 0.0 and dp is not None and dp != d and _native_attention_ok(qkv, dp):
        # head widths between the two kernel widths (80, 96, ...) run on the wider kernel over zero-padded heads
        wide = pad_fused_qkv(qkv, groups, qpg, d, dp)
        out = _FusedQKVAttentionFn.apply(wide, cu_seqlens.to(torch.int32), max_seqlen, groups, qpg, dp, scale, causal)
        return out.view(qkv.shape[0], groups * qpg, dp)[:, :, :d].reshape(qkv.shape[0], groups * qpg * d)
    note_fallback("attention", "attention dropout" if dropout_p != 0.0 else f"head_dim {d} or the strides of the fused projection", qkv)
    q, k, v = split_fused_qkv(qkv, groups, qpg, d)
    out = attention_varlen_reference(q, k, v, cu_seqlens, scale, causal, dropout_p)
    return out.reshape(qkv.shape[0], groups * qpg * d)

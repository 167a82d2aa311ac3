"""Recurrent scans (tanh RNN and GRU with per-head block-diagonal state transitions) on the sm_100a kernels of
``csrc/ops/recurrent.cu``: one CTA per (document, head), transition matrices resident in shared memory, packed
documents taken from ``cu_seqlens`` on the device (no host synchronisation). The PyTorch loops in
``lm_engine/hf_models/layers/recurrent.py`` are the reference and the fallback
(parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/{rnn.py:117-125, gru.py:122-134}, which call the
``rnn_cute`` / ``gru_cute`` kernels)."""

from __future__ import annotations

import torch

from . import native, native_available

_WIDTHS = (16, 32, 64, 128)


def recurrent_kernel_ok(x: torch.Tensor, state_head_dim: int) -> bool:
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and state_head_dim in _WIDTHS and native_available()
            and hasattr(native(), "recurrent_scan_fwd"))


class _RecurrentScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, h0, cu_seqlens, num_heads, head_dim, gru, clip):
        C = native()
        out, gates = C.recurrent_scan_fwd(x, weight, h0, cu_seqlens, num_heads, head_dim, gru)
        ctx.save_for_backward(out, gates, weight, h0 if h0 is not None else x.new_empty(0), cu_seqlens)
        ctx.meta = (num_heads, head_dim, gru, 0.0 if clip is None else float(clip), h0 is not None)
        return out

    @staticmethod
    def backward(ctx, d_out):
        out, gates, weight, h0, cu_seqlens = ctx.saved_tensors
        n, d, gru, clip, has_h0 = ctx.meta
        dx, dw, dh0 = native().recurrent_scan_bwd(d_out.contiguous(), out, gates, weight, h0 if has_h0 else None, cu_seqlens,
                                                  n, d, gru, clip)
        return dx, dw, (dh0 if has_h0 else None), None, None, None, None, None


def recurrent_scan(x: torch.Tensor, weight: torch.Tensor, cu_seqlens: torch.Tensor, num_heads: int, head_dim: int, gru: bool,
                   clip: float | None, h0: torch.Tensor | None = None) -> torch.Tensor:
    """``x``: ``[tokens, gates * num_heads * head_dim]`` (gates = 3 for the GRU in the order candidate, forget, reset;
    1 for the RNN); ``weight``: ``[gates * num_heads, head_dim, head_dim]``; ``cu_seqlens``: int32 document boundaries;
    ``h0``: optional initial state ``[documents, num_heads, head_dim]``. Returns all states ``[tokens, num_heads, head_dim]``."""
    if x.stride(-1) != 1:
        x = x.contiguous()
    w32 = weight.float().contiguous()
    h32 = None if h0 is None else h0.float().contiguous()
    return _RecurrentScan.apply(x, w32, h32, cu_seqlens, num_heads, head_dim, gru, clip)

"""Token-layout operators with sm_100a kernels (``csrc/ops/sequence.cu``) and plain PyTorch fallbacks:

``pack_sequence`` / ``unpack_sequence``  padded ``[batch, seq, ...]`` <-> packed ``[tokens, ...]`` (parity:
                                          lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/packing.py:28-56)
``causal_conv1d_packed``                  depthwise causal convolution over packed sequences, optional SiLU
``topk_route``                            router: top-k, softmax over the selected logits, expert histogram
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native, native_available


def _native_rows(x: torch.Tensor, lead: int) -> bool:
    row_bytes = x[(0,) * lead].numel() * x.element_size() if x.numel() else 0
    return native_available() and x.is_cuda and hasattr(native(), "pack_sequence") and row_bytes % 16 == 0 and row_bytes > 0


def _pack_torch(x, cu, left):
    b, s = x.shape[:2]
    lengths = (cu[1:] - cu[:-1]).long()
    pos = torch.arange(s, device=x.device).unsqueeze(0)
    mask = pos >= (s - lengths).unsqueeze(1) if left else pos < lengths.unsqueeze(1)
    return x[mask]


def _unpack_torch(x, cu, batch, seq, left):
    lengths = (cu[1:] - cu[:-1]).long()
    pos = torch.arange(seq, device=x.device).unsqueeze(0)
    mask = pos >= (seq - lengths).unsqueeze(1) if left else pos < lengths.unsqueeze(1)
    out = x.new_zeros((batch, seq, *x.shape[1:]))
    out[mask] = x
    return out


class _Pack(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu, left):
        ctx.save_for_backward(cu)
        ctx.shape, ctx.left = x.shape, left
        x = x.contiguous()
        if _native_rows(x, 2):
            return native().pack_sequence(x, cu, int(cu[-1].item()), left)
        return _pack_torch(x, cu, left)

    @staticmethod
    def backward(ctx, g):
        (cu,) = ctx.saved_tensors
        g = g.contiguous()
        if _native_rows(g, 1):
            return native().unpack_sequence(g, cu, ctx.shape[0], ctx.shape[1], ctx.left), None, None
        return _unpack_torch(g, cu, ctx.shape[0], ctx.shape[1], ctx.left), None, None


class _Unpack(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu, batch, seq, left):
        ctx.save_for_backward(cu)
        ctx.left = left
        x = x.contiguous()
        if _native_rows(x, 1):
            return native().unpack_sequence(x, cu, batch, seq, left)
        return _unpack_torch(x, cu, batch, seq, left)

    @staticmethod
    def backward(ctx, g):
        (cu,) = ctx.saved_tensors
        g = g.contiguous()
        if _native_rows(g, 2):
            return native().pack_sequence(g, cu, int(cu[-1].item()), ctx.left), None, None, None, None
        return _pack_torch(g, cu, ctx.left), None, None, None, None


def compute_cu_seqlens_and_max_seqlen_from_attention_mask(attention_mask: torch.Tensor) -> tuple[torch.Tensor, int]:
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    cu_seqlens = F.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
    return cu_seqlens, int(seqlens.max().item())


def pack_sequence(inputs, cu_seqlens: torch.Tensor, padding_side: str = "left"):
    """``[batch, seq, ...] -> [tokens, ...]``: the real tokens of every row, rows one after the other."""
    if isinstance(inputs, (list, tuple)):
        return [pack_sequence(x, cu_seqlens, padding_side) for x in inputs]
    return _Pack.apply(inputs, cu_seqlens.to(torch.int32), padding_side == "left")


def unpack_sequence(inputs, cu_seqlens: torch.Tensor, desired_shape: tuple[int, ...], padding_side: str = "left"):
    """Inverse of :func:`pack_sequence`; padding positions are zero. ``desired_shape = (batch, seq, ...)``."""
    if isinstance(inputs, (list, tuple)):
        return [unpack_sequence(x, cu_seqlens, desired_shape, padding_side) for x in inputs]
    return _Unpack.apply(inputs, cu_seqlens.to(torch.int32), desired_shape[0], desired_shape[1], padding_side == "left")


# ----------------------------------------------------------------------------------------------------------------------
def _conv_torch(x, weight, bias, cu, silu):
    k = weight.shape[-1]
    pieces = []
    bounds = cu.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e > s:
            seq = F.pad(x[s:e].t().unsqueeze(0), (k - 1, 0))
            pieces.append(F.conv1d(seq, weight.view(-1, 1, k).to(x.dtype), None if bias is None else bias.to(x.dtype), groups=x.shape[1]).squeeze(0).t())
    y = torch.cat(pieces, dim=0) if pieces else x.new_zeros(x.shape)
    return F.silu(y) if silu else y


class _CausalConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, cu, silu):
        w32 = weight.reshape(weight.shape[0], -1).float().contiguous()
        b32 = None if bias is None else bias.float().contiguous()
        ctx.save_for_backward(x, w32, b32 if b32 is not None else x.new_empty(0), cu)
        ctx.has_bias, ctx.silu, ctx.w_shape, ctx.w_dtype = bias is not None, silu, weight.shape, weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        return native().causal_conv1d_fwd(x.contiguous(), w32, b32, cu, silu)

    @staticmethod
    def backward(ctx, dy):
        x, w32, b32, cu = ctx.saved_tensors
        dx, dw, db = native().causal_conv1d_bwd(dy.contiguous(), x.contiguous(), w32, b32 if ctx.has_bias else None, cu, ctx.silu)
        return dx, dw.view(ctx.w_shape).to(ctx.w_dtype), db.to(ctx.b_dtype) if ctx.has_bias else None, None, None


def causal_conv1d_packed(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, cu_seqlens: torch.Tensor,
                         activation: str | None = None) -> torch.Tensor:
    """Depthwise causal convolution of packed sequences: ``x [tokens, channels]``, ``weight [channels, 1, K]`` (or
    ``[channels, K]``); the window never reaches into the previous sequence. ``activation``: None or "silu"."""
    assert activation in (None, "silu", "swish")
    silu = activation is not None
    cu = cu_seqlens.to(torch.int32)
    if (native_available() and x.is_cuda and hasattr(native(), "causal_conv1d_fwd") and x.dtype in (torch.bfloat16, torch.float32)
            and weight.shape[-1] <= 8 and x.dim() == 2):
        return _CausalConv.apply(x, weight, bias, cu, silu)
    return _conv_torch(x, weight.reshape(weight.shape[0], -1), bias, cu, silu)


# ----------------------------------------------------------------------------------------------------------------------
class _TopKRoute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, want_counts):
        weights, experts, counts = native().topk_route(logits.contiguous(), k, want_counts)
        ctx.save_for_backward(weights, experts)
        ctx.shape, ctx.dtype = logits.shape, logits.dtype
        ctx.mark_non_differentiable(experts, counts)
        return weights, experts, counts

    @staticmethod
    def backward(ctx, d_weights, _e, _c):
        weights, experts = ctx.saved_tensors
        inner = (d_weights * weights).sum(dim=-1, keepdim=True)
        d_top = weights * (d_weights - inner)  # softmax backward over the k selected logits
        d_logits = torch.zeros(ctx.shape, dtype=torch.float32, device=d_weights.device)
        d_logits.scatter_(1, experts.long(), d_top)
        return d_logits.to(ctx.dtype), None, None


def topk_route(logits: torch.Tensor, k: int, want_counts: bool = False):
    """``(weights fp32 [tokens, k], experts int64 [tokens, k], counts int32 [experts] or None)``: the ``k`` largest
    logits of every token, a softmax over just those, and how many tokens picked each expert."""
    tokens, num_experts = logits.shape
    if (native_available() and logits.is_cuda and hasattr(native(), "topk_route") and num_experts <= 256 and k <= 8
            and logits.dtype in (torch.bfloat16, torch.float32)):
        weights, experts, counts = _TopKRoute.apply(logits, k, want_counts)
        return weights, experts.long(), (counts if want_counts else None)
    top, experts = (logits.max(dim=-1, keepdim=True) if k == 1 else logits.topk(k, dim=-1))
    weights = F.softmax(top.float(), dim=-1)
    counts = torch.bincount(experts.flatten(), minlength=num_experts).to(torch.int32) if want_counts else None
    return weights, experts, counts

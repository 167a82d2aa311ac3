"""Mamba-2 selective state-space recurrence on the state-resident scan kernel of ``csrc/ops/ssd_scan.cu``
(the role of ``mamba_chunk_scan_combined`` for the reference, lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/
mamba2.py:461-504 there). ``lm_engine.hf_models.layers.mamba2.ssd_chunk_scan`` is the PyTorch formulation of the same
function and the fallback.

    h_t = exp(a_t) h_{t-1} + x_t b_t^T,   y_t = h_t c_t        x: [B, L, H, P], a: [B, L, H], b / c: [B, L, G, N]

Forward is one scan; backward is three more scans of the same kernel (the transposed state for dc, the adjoint state
backwards in time for dx and db) and a reversed cumulative sum for da: ``da_t = <dy_t, y_t> - <x_t, dx_t> + da_{t+1}``.
"""

from __future__ import annotations

import torch

from . import native, native_available


def ssd_kernel_ok(x: torch.Tensor, state_size: int) -> bool:
    if not (x.is_cuda and native_available() and hasattr(native(), "ssd_scan")):
        return False
    p = x.shape[-1]
    return p % 4 == 0 and state_size % 4 == 0 and p <= 256 and state_size <= 256


def _scan_reference(u, v, w, a, s0, reverse: bool):
    """The recurrence of the kernel, step by step in PyTorch (CPU path and oracle): ``s = decay * s + u_t v_t^T``,
    ``out_t = s w_t`` with the decay of step t forwards and of step t + 1 backwards."""
    B, L, H = a.shape
    expand = lambda t: t if t.shape[2] == H else t.repeat_interleave(H // t.shape[2], dim=2)
    u, v, w = expand(u), expand(v), expand(w)
    state = u.new_zeros(B, H, u.shape[-1], v.shape[-1]) if s0 is None else s0.clone()
    out = u.new_empty(B, L, H, u.shape[-1])
    decay_next = a.new_ones(B, H)
    for step in range(L):
        t = L - 1 - step if reverse else step
        decay_t = torch.exp(a[:, t])
        decay = decay_next if reverse else decay_t
        decay_next = decay_t
        state = decay[..., None, None] * state + u[:, t, :, :, None] * v[:, t, :, None, :]
        out[:, t] = torch.einsum("bhqr,bhr->bhq", state, w[:, t])
    return out, state


def _scan(u, v, w, a, s0, reverse: bool):
    if u.is_cuda and native_available() and hasattr(native(), "ssd_scan"):
        return native().ssd_scan(u, v, w, a, s0, reverse)
    return _scan_reference(u, v, w, a, s0, reverse)


_SIDE_STREAMS: dict[torch.device, tuple[torch.cuda.Stream, torch.cuda.Stream]] = {}


def _side_streams(device: torch.device):
    if device not in _SIDE_STREAMS:
        _SIDE_STREAMS[device] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _SIDE_STREAMS[device]


class _SSDScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, a, b, c, h0, cu_seqlens):
        starts = None
        if cu_seqlens is not None:
            # packed documents in one row: a decay of exp(-inf) = 0 at the first token of a document resets the state
            # there (forwards) and cuts the adjoint state (backwards); no host round trip for the boundaries
            assert x.shape[0] == 1, "packed documents come as one row of tokens"
            L = x.shape[1]
            starts = torch.zeros(L + 1, dtype=torch.bool, device=x.device)
            starts[cu_seqlens[:-1].long()] = True
            starts = starts[:L]
            a = a.masked_fill(starts[None, :, None], float("-inf"))
        y, final = _scan(x, b, c, a, h0, False)
        empty = x.new_empty(0)
        ctx.save_for_backward(x, a, b, c, y, final, h0 if h0 is not None else empty,
                              cu_seqlens if cu_seqlens is not None else empty, starts if starts is not None else empty)
        ctx.has_h0 = h0 is not None
        ctx.packed = cu_seqlens is not None
        return y, final

    @staticmethod
    def backward(ctx, dy, dfinal):
        x, a, b, c, y, final, h0, cu_seqlens, starts = ctx.saved_tensors
        B, L, H, P = x.shape
        G, N = b.shape[2], b.shape[3]
        dy = dy.contiguous() if dy is not None else torch.zeros_like(y)
        h0 = h0 if ctx.has_h0 else None
        dfinal = None if dfinal is None else dfinal.contiguous()
        transposed = lambda s: None if s is None else s.transpose(-1, -2).contiguous()
        h0_t, dfinal_t = transposed(h0), transposed(dfinal)
        if x.is_cuda:
            # three independent scans of one CTA per (batch, head) each: side streams let them share the SMs
            main = torch.cuda.current_stream(x.device)
            side = _side_streams(x.device)
            for stream in side:
                stream.wait_stream(main)
            with torch.cuda.stream(side[0]):
                dc_heads, _ = _scan(b, x, dy, a, h0_t, False)
            with torch.cuda.stream(side[1]):
                db_heads, _ = _scan(c, dy, x, a, dfinal_t, True)
            dx, adjoint0 = _scan(dy, c, b, a, dfinal, True)
            for stream, result in zip(side, (dc_heads, db_heads)):
                main.wait_stream(stream)
                result.record_stream(main)
        else:
            dc_heads, _ = _scan(b, x, dy, a, h0_t, False)
            db_heads, _ = _scan(c, dy, x, a, dfinal_t, True)
            dx, adjoint0 = _scan(dy, c, b, a, dfinal, True)
        r = (dy * y).sum(-1) - (x * dx).sum(-1)
        da = torch.flip(torch.cumsum(torch.flip(r, dims=[1]), dim=1), dims=[1])
        tail = None if dfinal is None else (dfinal * final).sum(dim=(-1, -2))[:, None, :]
        if ctx.packed:
            # the sum runs to the end of the token's own document: subtract what lies beyond it
            bounds = cu_seqlens.long()
            document = torch.bucketize(torch.arange(L, device=x.device), bounds[1:], right=True).clamp(max=bounds.numel() - 2)
            next_start = bounds[document + 1]
            beyond = torch.cat([da, da.new_zeros(B, 1, H)], dim=1)[:, next_start]
            da = da - beyond
            if tail is not None:
                da = da + tail * (next_start == L)[None, :, None]
            da = da.masked_fill(starts[None, :, None], 0.0)
        elif tail is not None:
            da = da + tail
        db = db_heads.view(B, L, G, H // G, N).sum(3)
        dc = dc_heads.view(B, L, G, H // G, N).sum(3)
        dh0 = torch.exp(a[:, 0])[..., None, None] * adjoint0 if ctx.has_h0 else None
        return dx, da, db, dc, dh0, None


def ssd_scan(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, initial_state: torch.Tensor | None = None,
             cu_seqlens: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [B, L, H, P]`` (already multiplied by dt), ``a [B, L, H]`` (= A * dt), ``b`` / ``c`` ``[B, L, G, N]`` with
    ``G`` dividing ``H``. Returns ``(y [B, L, H, P], final_state [B, H, P, N])``, all fp32. With ``cu_seqlens`` the single
    row (``B = 1``) holds packed documents and the state starts from zero at every document."""
    f32 = lambda t: None if t is None else t.float().contiguous()
    return _SSDScan.apply(f32(x), f32(a), f32(b), f32(c), f32(initial_state), cu_seqlens)

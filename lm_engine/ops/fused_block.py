"""Whole-block forward/backward for the common dense decoder block on packed sequences:

    h  = x + c_proj(attention(rope(c_attn(rmsnorm(x)))))
    y  = h + mlp.c_proj(swiglu(mlp.c_fc(rmsnorm(h))))

executed as an explicit schedule of this library's kernels instead of an autograd trace. Only the tensors that
cannot be recomputed cheaply are kept for backward (block input, fused qkv after RoPE, attention output + lse,
mid-block residual, c_fc output, two per-token rstd vectors: about 47k bf16 values per token for the 8B shape);
the two normalised activations and the SwiGLU output are recomputed. Weight gradients are accumulated by the
GEMM epilogue directly into the fp32 ``main_grad`` buffers of the sharded-training engine when those exist.
"""

from __future__ import annotations

import torch

from . import _weight_grad_target, native, status_word
from .timeline import site


def _wgrad(C, dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, st):
    """dW = dy^T x. Accumulates into ``weight.main_grad`` when present (returns None), else returns the gradient."""
    target = _weight_grad_target(weight)
    if target is not None:
        C.gemm(dy, x, target.view(weight.shape), True, True, True, 1.0, st, 0)
        return None
    dw = torch.empty(weight.shape, device=weight.device, dtype=torch.float32)
    C.gemm(dy, x, dw, True, True, False, 1.0, st, 0)
    return dw.to(weight.dtype)


def _norm_wgrad_buffer(weight: torch.Tensor):
    target = _weight_grad_target(weight)
    if target is not None:
        return target.view(-1), True
    return torch.empty(weight.numel(), device=weight.device, dtype=torch.float32), False


class FusedDenseBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ln1_w, w_qkv, w_o, ln2_w, w_fc, w_proj, cos, sin, position_ids, cu_seqlens, max_seqlen,
                groups, qpg, head_dim, rope_dim, softmax_scale, eps):
        C = native()
        st = status_word(x.device)
        T, H = x.shape
        with site("fwd.ln1"):
            n1, rstd1 = C.rmsnorm_fwd(x, None, ln1_w, eps, False)
        qkv = torch.empty(T, w_qkv.shape[0], device=x.device, dtype=x.dtype)
        with site("fwd.c_attn"):
            C.gemm(n1, w_qkv, qkv, False, False, False, 1.0, st, 0)
        del n1
        if rope_dim > 0:
            with site("fwd.rope"):
                C.rope_(qkv, cos, sin, position_ids, groups, qpg, head_dim, rope_dim, False)
        with site("fwd.attention"):
            attn, lse = C.attn_fwd(qkv, cu_seqlens, max_seqlen, groups, qpg, head_dim, softmax_scale, True, st)
        a = torch.empty(T, H, device=x.device, dtype=x.dtype)
        with site("fwd.attn_c_proj"):
            C.gemm(attn, w_o, a, False, False, False, 1.0, st, 0)
        with site("fwd.residual+ln2"):
            n2, rstd2, h = C.rmsnorm_fwd(a, x, ln2_w, eps, True)
        del a
        fc = torch.empty(T, w_fc.shape[0], device=x.device, dtype=x.dtype)
        inter = w_fc.shape[0] // 2
        if inter % 128 == 0 and T >= 256:
            # up-projection with the activation in its epilogue: fc is written for backward, never read back here
            act = torch.empty(T, inter, device=x.device, dtype=x.dtype)
            with site("fwd.c_fc+swiglu"):
                C.gemm_swiglu(n2, w_fc, fc, act, st)
        else:
            with site("fwd.c_fc"):
                C.gemm(n2, w_fc, fc, False, False, False, 1.0, st, 0)
            with site("fwd.swiglu"):
                act = C.swiglu_fwd(fc)
        del n2
        m = torch.empty(T, H, device=x.device, dtype=x.dtype)
        with site("fwd.mlp_c_proj"):
            C.gemm(act, w_proj, m, False, False, False, 1.0, st, 0)
        del act
        with site("fwd.residual_add"):
            y = C.add_bf16(h, m)
        ctx.save_for_backward(x, rstd1, qkv, attn, lse, h, rstd2, fc, ln1_w, w_qkv, w_o, ln2_w, w_fc, w_proj, cos, sin,
                              position_ids, cu_seqlens)
        ctx.meta = (max_seqlen, groups, qpg, head_dim, rope_dim, softmax_scale, eps)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x, rstd1, qkv, attn, lse, h, rstd2, fc, ln1_w, w_qkv, w_o, ln2_w, w_fc, w_proj, cos, sin, position_ids,
         cu_seqlens) = ctx.saved_tensors
        max_seqlen, groups, qpg, head_dim, rope_dim, softmax_scale, eps = ctx.meta
        C = native()
        st = status_word(x.device)
        T, H = x.shape
        dy = dy.contiguous()

        # ---- MLP
        inter = w_proj.shape[1]
        if hasattr(C, "gemm_swiglu_bwd") and inter % 64 == 0 and T >= 256:
            # data gradient of the down-projection with the SwiGLU backward in its epilogue: d(act) never reaches memory
            dfc = torch.empty(T, 2 * inter, device=x.device, dtype=x.dtype)
            act = torch.empty(T, inter, device=x.device, dtype=x.dtype)
            with site("bwd.mlp_c_proj.dgrad+swiglu"):
                C.gemm_swiglu_bwd(dy, w_proj, fc, dfc, act, st)
        else:
            dact = torch.empty(T, inter, device=x.device, dtype=x.dtype)
            with site("bwd.mlp_c_proj.dgrad"):
                C.gemm(dy, w_proj, dact, False, True, False, 1.0, st, 0)
            with site("bwd.swiglu"):
                dfc, act = C.swiglu_bwd(dact, fc, True)
            del dact
        with site("bwd.mlp_c_proj.wgrad"):
            g_proj = _wgrad(C, dy, act, w_proj, st)
        del act
        with site("bwd.ln2.recompute"):
            n2, _ = C.rmsnorm_fwd(h, None, ln2_w, eps, False)
        with site("bwd.c_fc.wgrad"):
            g_fc = _wgrad(C, dfc, n2, w_fc, st)
        del n2
        dn2 = torch.empty(T, H, device=x.device, dtype=x.dtype)
        with site("bwd.c_fc.dgrad"):
            C.gemm(dfc, w_fc, dn2, False, True, False, 1.0, st, 0)
        del dfc
        buf2, acc2 = _norm_wgrad_buffer(ln2_w)
        with site("bwd.ln2"):
            dh = C.rmsnorm_bwd(dn2, h, ln2_w, rstd2, dy, buf2, acc2)
        del dn2

        # ---- attention
        dattn = torch.empty(T, w_o.shape[1], device=x.device, dtype=x.dtype)
        with site("bwd.attn_c_proj.dgrad"):
            C.gemm(dh, w_o, dattn, False, True, False, 1.0, st, 0)
        with site("bwd.attn_c_proj.wgrad"):
            g_o = _wgrad(C, dh, attn, w_o, st)
        with site("bwd.attention"):
            dqkv = C.attn_bwd(dattn, qkv, attn, lse, cu_seqlens, max_seqlen, groups, qpg, head_dim, softmax_scale, True, st)
        del dattn
        if rope_dim > 0:
            with site("bwd.rope"):
                C.rope_(dqkv, cos, sin, position_ids, groups, qpg, head_dim, rope_dim, True)
        with site("bwd.ln1.recompute"):
            n1, _ = C.rmsnorm_fwd(x, None, ln1_w, eps, False)
        with site("bwd.c_attn.wgrad"):
            g_qkv = _wgrad(C, dqkv, n1, w_qkv, st)
        del n1
        dn1 = torch.empty(T, H, device=x.device, dtype=x.dtype)
        with site("bwd.c_attn.dgrad"):
            C.gemm(dqkv, w_qkv, dn1, False, True, False, 1.0, st, 0)
        del dqkv
        buf1, acc1 = _norm_wgrad_buffer(ln1_w)
        with site("bwd.ln1"):
            dx = C.rmsnorm_bwd(dn1, x, ln1_w, rstd1, dh, buf1, acc1)

        # every gradient of this block is in place: under sharded data parallelism the block's reduce-scatter may start
        unit = getattr(w_qkv, "_lm_engine_unit", None)
        if unit is not None and acc1 and acc2 and getattr(unit, "engine", None) is not None:
            unit.engine.unit_backward_done(unit)

        g_ln1 = None if acc1 else buf1.to(ln1_w.dtype)
        g_ln2 = None if acc2 else buf2.to(ln2_w.dtype)
        return (dx, g_ln1, g_qkv, g_o, g_ln2, g_fc, g_proj) + (None,) * 11


def fused_dense_block(x, ln1_w, w_qkv, w_o, ln2_w, w_fc, w_proj, cos, sin, position_ids, cu_seqlens, max_seqlen,
                      groups, qpg, head_dim, rope_dim, softmax_scale, eps) -> torch.Tensor:
    return FusedDenseBlockFn.apply(x, ln1_w, w_qkv, w_o, ln2_w, w_fc, w_proj, cos, sin, position_ids, cu_seqlens,
                                   int(max_seqlen), groups, qpg, head_dim, rope_dim, float(softmax_scale), float(eps))

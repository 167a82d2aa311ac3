"""8-bit floating point training of the linear layers (API parity: lm_engine/fp8.py:51-101).

The reference converts linears with ``torchao.float8`` (one dynamic scale per tensor). Here the same numerics run on
this engine's own kernels: per-tensor dynamic scaling, e4m3 for activations and weights, e5m2 for output gradients,
fp32 accumulation in the tcgen05 ``kind::f8f6f4`` GEMM (``csrc/gemm/gemm_fp8.cu``), which reads K-major and MN-major
operands, so the forward, data-gradient and weight-gradient products use the same three quantised tensors and no
transposed copies.

``fp8_recipe: mxfp8`` selects the OCP microscaling format instead: e4m3 payload with one power-of-two (E8M0) scale per 32
consecutive elements along the contraction dimension of each product. On the GPU a quantisation kernel writes payload
and scale codes (the latter in the tile layout the tensor core reads) and the products run on the block-scaled tcgen05
GEMM (``tcgen05.mma.kind::mxf8f6f4.block_scale``, ``csrc/gemm/gemm_mxfp8.cu``): forward with blocks along the input
features of activations and weights, data gradient with blocks along the output features (the weight read MN-major),
weight gradient with blocks along the tokens (both operands read MN-major), i.e. every tensor is quantised once per
direction it is contracted along. Sizes that are not multiples of 128, and CPU tensors, take the PyTorch restatement
of the same format (quantise, dequantise, multiply), which is also the numerical oracle of the kernels.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import ops

E4M3, E5M2 = 0, 1


def quantize(x: torch.Tensor, fmt: int = E4M3) -> tuple[torch.Tensor, torch.Tensor]:
    """``(uint8 payload shaped like x, fp32 device scalar to multiply back with)``; no host synchronisation."""
    x = x.contiguous()
    amax = x.abs().amax().float().reshape(1)
    q, scale_inv = ops.native().quantize_fp8(x if x.dtype == torch.bfloat16 else x.bfloat16(), amax, fmt)
    return q, scale_inv


def dequantize(q: torch.Tensor, scale_inv: torch.Tensor, fmt: int = E4M3) -> torch.Tensor:
    dtype = torch.float8_e4m3fn if fmt == E4M3 else torch.float8_e5m2
    return q.view(dtype).float() * scale_inv


MX_BLOCK = 32
_E4M3_MAX = 448.0
_E4M3_EMAX = 8  # 2^8 is the largest power of two that e4m3 represents


def mx_quantize(x: torch.Tensor, dim: int = -1) -> tuple[torch.Tensor, torch.Tensor]:
    """OCP MXFP8 (e4m3) along ``dim``: ``(payload float8_e4m3fn shaped like x, scales uint8 = biased E8M0 exponents with
    the size of ``dim`` divided by 32)``. The shared exponent of a block is ``floor(log2(amax)) - 8``; values are rounded to
    nearest even and saturate at +-448."""
    x = x.movedim(dim, -1)
    assert x.shape[-1] % MX_BLOCK == 0, "the quantised dimension must be a multiple of 32"
    blocks = x.float().reshape(*x.shape[:-1], x.shape[-1] // MX_BLOCK, MX_BLOCK)
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    exponent = torch.floor(torch.log2(amax.clamp(min=2.0**-126))) - _E4M3_EMAX
    exponent = exponent.clamp(-127, 127)
    scaled = (blocks * torch.exp2(-exponent)).clamp(-_E4M3_MAX, _E4M3_MAX)
    payload = scaled.to(torch.float8_e4m3fn).reshape(x.shape).movedim(-1, dim)
    scales = (exponent.squeeze(-1) + 127).to(torch.uint8).movedim(-1, dim)
    return payload, scales


def mx_dequantize(payload: torch.Tensor, scales: torch.Tensor, dim: int = -1, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    p = payload.movedim(dim, -1).float()
    e = scales.movedim(dim, -1).float() - 127
    out = p.reshape(*p.shape[:-1], p.shape[-1] // MX_BLOCK, MX_BLOCK) * torch.exp2(e).unsqueeze(-1)
    return out.reshape(p.shape).movedim(-1, dim).to(dtype)


def _mx_round_trip(x: torch.Tensor, dim: int) -> torch.Tensor:
    return mx_dequantize(*mx_quantize(x, dim), dim=dim, dtype=x.dtype)


class _MXLinear(torch.autograd.Function):
    """Linear layer with MXFP8 operands: every product quantises both operands in blocks of 32 along its own contraction
    dimension (features for the forward product, output features for the data gradient, tokens for the weight gradient)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.shape, ctx.has_bias = shape, bias is not None
        y = ops.linear(_mx_round_trip(x2, 1), _mx_round_trip(weight, 1), bias)
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = _mx_round_trip(dy2, 1) @ _mx_round_trip(weight, 0)        # contraction over the output features
        dw = _mx_round_trip(dy2, 0).t() @ _mx_round_trip(x2, 0)        # contraction over the tokens
        db = dy2.sum(0) if ctx.has_bias else None
        return dx.view(ctx.shape), dw.to(weight.dtype), db


class _MXLinearNative(torch.autograd.Function):
    """The same three products on the block-scaled GEMM. ``quantize_mx(t, along_rows)`` quantises a row-major matrix in
    blocks of 32 along its columns (``False``) or along its rows (``True``) and returns payload and tiled scale codes."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        C, st = ops.native(), ops.status_word(x.device)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        xq, xs = C.quantize_mx(x2, False, E4M3)
        wq, ws = C.quantize_mx(weight.contiguous(), False, E4M3)
        y = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        C.gemm_mxfp8(xq, xs, wq, ws, y, False, False, E4M3, E4M3, False, 1.0, st)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x2)
        ctx.weight, ctx.shape, ctx.has_bias = weight, shape, bias is not None
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        weight = ctx.weight
        C, st = ops.native(), ops.status_word(dy.device)
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        # dx[T, in] = dy[T, out] . W[out, in]: blocks along the output features; W read MN-major
        gq, gs = C.quantize_mx(dy2, False, E4M3)
        wq, ws = C.quantize_mx(weight.contiguous(), True, E4M3)
        dx = torch.empty(dy2.shape[0], weight.shape[1], dtype=torch.bfloat16, device=dy.device)
        C.gemm_mxfp8(gq, gs, wq, ws, dx, False, True, E4M3, E4M3, False, 1.0, st)
        # dW[out, in] = dy^T . x: blocks along the tokens; both read MN-major; accumulated into the fp32 main gradient
        # when the engine provides one
        gq, gs = C.quantize_mx(dy2, True, E4M3)
        xq, xs = C.quantize_mx(x2, True, E4M3)
        target = getattr(weight, "main_grad", None)
        if target is not None:
            C.gemm_mxfp8(gq, gs, xq, xs, target, True, True, E4M3, E4M3, True, 1.0, st)
            dw = None
        else:
            dw32 = torch.empty(weight.shape, dtype=torch.float32, device=dy.device)
            C.gemm_mxfp8(gq, gs, xq, xs, dw32, True, True, E4M3, E4M3, False, 1.0, st)
            dw = dw32.to(weight.dtype)
        db = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx.view(ctx.shape), dw, db


def _mx_native_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    tokens = x.numel() // x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and ops.native_available()
            and hasattr(ops.native(), "gemm_mxfp8") and tokens % 128 == 0 and weight.shape[0] % 128 == 0 and weight.shape[1] % 128 == 0)


def mx_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if _mx_native_ok(x, weight):
        return _MXLinearNative.apply(x, weight, bias)
    ops.note_fallback("mx_linear", "token count or feature sizes are not multiples of 128", x, weight)
    return _MXLinear.apply(x, weight, bias)


class _FP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        C, st = ops.native(), ops.status_word(x.device)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        xq, xs = quantize(x2, E4M3)
        wq, ws = quantize(weight, E4M3)
        y = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        C.gemm_fp8(xq, wq, y, False, False, E4M3, E4M3, False, 1.0, xs, ws, st)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(xq, xs, wq, ws)
        ctx.weight, ctx.shape, ctx.has_bias = weight, shape, bias is not None
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xq, xs, wq, ws = ctx.saved_tensors
        weight = ctx.weight
        C, st = ops.native(), ops.status_word(dy.device)
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        gq, gs = quantize(dy2, E5M2)
        # dx[T, in] = dy[T, out] . W[out, in]: W read MN-major
        dx = torch.empty(dy2.shape[0], weight.shape[1], dtype=torch.bfloat16, device=dy.device)
        C.gemm_fp8(gq, wq, dx, False, True, E5M2, E4M3, False, 1.0, gs, ws, st)
        # dW[out, in] = dy^T . x: both read MN-major; accumulated into the fp32 main gradient when the engine provides one
        target = getattr(weight, "main_grad", None)
        if target is not None:
            C.gemm_fp8(gq, xq, target, True, True, E5M2, E4M3, True, 1.0, gs, xs, st)
            dw = None
        else:
            dw32 = torch.empty(weight.shape, dtype=torch.float32, device=dy.device)
            C.gemm_fp8(gq, xq, dw32, True, True, E5M2, E4M3, False, 1.0, gs, xs, st)
            dw = dw32.to(weight.dtype)
        db = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx.view(ctx.shape), dw, db


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    return _FP8Linear.apply(x, weight, bias)


def _eligible(module: nn.Module) -> bool:
    return isinstance(module, nn.Linear) and module.in_features % 16 == 0 and module.out_features % 16 == 0


class FP8Manager:
    """Switches the linear layers of every model of a container to fp8 GEMMs (the output projection / LM head stays in
    bf16, like in the reference). The scaling-type arguments are accepted for compatibility; scaling is dynamic."""

    def __init__(self, model_container, enable_fsdp_fp8_all_gather: bool = False, precompute_fp8_dynamic_scale_for_fsdp: bool = False,
                 torch_compile: bool = False, scaling_type_input=None, scaling_type_weight=None, scaling_type_grad_output=None,
                 recipe: str = "tensorwise") -> None:
        assert recipe in ("tensorwise", "mxfp8"), recipe
        if recipe == "tensorwise" and (not ops.native_available() or not hasattr(ops.native(), "gemm_fp8")):
            raise RuntimeError("tensor-scaled fp8 training needs the sm_100a extension")
        self.recipe = recipe
        forward = _fp8_forward if recipe == "tensorwise" else _mx_forward
        self.converted = 0
        for model in model_container:
            for name, module in model.named_modules():
                if hasattr(module, "_fusable"):
                    module._fusable = False  # the whole-block bf16 schedule would bypass the converted linears
                if _eligible(module) and not name.endswith(("lm_head", "output")):
                    module.forward = forward.__get__(module, type(module))
                    self.converted += 1
                elif type(module).__name__ in ("ColumnParallelLinear", "RowParallelLinear") and not name.endswith(("lm_head", "output")):
                    # tensor-parallel linears keep their collectives and hand the local product to the recipe
                    module.linear_function = _tp_product(recipe)
                    self.converted += 1

    @staticmethod
    def precompute_float8_dynamic_scale_for_fsdp(model_container) -> None:
        """Nothing to do: weights are quantised from the gathered bf16 copy when they are used."""

    @staticmethod
    def sync_float8_amax_and_scale_history(model_container) -> None:
        """Nothing to do: scaling is dynamic (no amax history)."""


def _tp_product(recipe: str):
    def product(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        tokens = x.numel() // x.shape[-1]
        if recipe == "mxfp8":
            if tokens % MX_BLOCK == 0 and weight.shape[0] % MX_BLOCK == 0 and weight.shape[1] % MX_BLOCK == 0:
                return mx_linear(x, weight, bias)
        elif x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and tokens % 16 == 0 and weight.shape[0] % 16 == 0 \
                and weight.shape[1] % 16 == 0:
            return fp8_linear(x, weight, bias)
        return ops.linear(x, weight, bias)

    return product


def _fp8_forward(self, x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and x.numel() // x.shape[-1] % 16 == 0:
        return fp8_linear(x, self.weight, self.bias)
    return ops.linear(x, self.weight, self.bias)


def _mx_forward(self, x: torch.Tensor) -> torch.Tensor:
    tokens = x.numel() // x.shape[-1]
    if tokens % MX_BLOCK == 0 and self.in_features % MX_BLOCK == 0 and self.out_features % MX_BLOCK == 0:
        return mx_linear(x, self.weight, self.bias)
    return ops.linear(x, self.weight, self.bias)

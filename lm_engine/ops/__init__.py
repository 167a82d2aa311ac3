"""Operator layer: every hot op as (a) an autograd function over the sm_100a kernels in ``csrc/`` and (b) a plain
PyTorch restatement that serves as CPU path and numerical oracle.

The native path is taken for CUDA bf16 tensors when the extension is built; anything else runs the PyTorch
restatement. If a CUDA device is present but the extension is missing, ``require_native()`` raises instead of
silently falling back.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .build import is_extension_built, load_extension
from .timeline import site

_C = None
_STATUS: dict[int, torch.Tensor] = {}


def native() :
    """The loaded extension module (built on demand when a CUDA device is present)."""
    global _C
    if _C is None:
        _C = load_extension()
    return _C


def native_available() -> bool:
    return torch.cuda.is_available() and is_extension_built()


def require_native() -> None:
    if torch.cuda.is_available() and not is_extension_built():
        raise RuntimeError("a CUDA device is present but the sm_100a extension is not built; run __graft_entry__.build()")


def use_native(*tensors: torch.Tensor) -> bool:
    if not native_available():
        return False
    return all(t is None or (t.is_cuda and t.dtype in (torch.bfloat16, torch.float32, torch.int32, torch.int64)) for t in tensors) and any(
        t is not None and t.dtype == torch.bfloat16 for t in tensors
    )


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels raise when a bounded wait runs out (0 = healthy)."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _STATUS:
        _STATUS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return _STATUS[index]


STATUS_GRAD_SCALE_MISMATCH = 6  # fused linear + cross entropy: upstream gradient differs from the promised scale


def check_status() -> None:
    """Host-side check of the status words (synchronises); raises if any kernel reported a timeout or a violated
    assumption."""
    for index, word in _STATUS.items():
        code = int(word.item())
        if code != 0:
            word.zero_()
            if code == STATUS_GRAD_SCALE_MISMATCH:
                raise RuntimeError(f"cuda:{index}: the fused linear + cross entropy was promised a gradient scale "
                                   "(grad_scale_hint) that differs from the gradient it received; its weight and input "
                                   "gradients of the steps since the last check are wrong")
            raise RuntimeError(f"a kernel on cuda:{index} gave up waiting (status {code})")


# ----------------------------------------------------------------------------- fallbacks are never silent
_STRICT = False
_FALLBACKS: dict[str, int] = {}
_WARNED: set[str] = set()


def set_strict(on: bool = True) -> None:
    """Strict mode: an op that would leave the sm_100a kernels for the PyTorch restatement on CUDA bf16 tensors raises
    instead (``kernel_args.strict`` in the YAML, ``LM_ENGINE_STRICT=1`` in the environment; the benchmark and the GPU
    tests run with it)."""
    global _STRICT
    _STRICT = bool(on)


def is_strict() -> bool:
    import os

    return _STRICT or os.environ.get("LM_ENGINE_STRICT", "0") == "1"


def note_fallback(site: str, reason: str, *tensors: torch.Tensor) -> None:
    """Called where an op takes the PyTorch path. On a machine with the native kernels and CUDA bf16 operands that is
    a lost kernel: it is counted (``fallback_counts()``), logged once per site and reason, and an error in strict mode.
    CPU tensors and other dtypes take the PyTorch path by design and are not reported."""
    if not native_available():
        return
    if not any(t is not None and t.is_cuda and t.dtype == torch.bfloat16 for t in tensors):
        return
    key = f"{site}: {reason}"
    _FALLBACKS[key] = _FALLBACKS.get(key, 0) + 1
    if is_strict():
        raise RuntimeError(f"strict mode: {site} would run the PyTorch path instead of its sm_100a kernel ({reason})")
    if key not in _WARNED:
        _WARNED.add(key)
        import logging

        logging.getLogger(__name__).warning(f"{site} runs the PyTorch path instead of its sm_100a kernel ({reason}); reported once")


def fallback_counts() -> dict[str, int]:
    """``{"site: reason": visits}`` of every op call that left the native kernels since the process started."""
    return dict(_FALLBACKS)


def launch_count() -> int:
    return int(native().launch_count()) if native_available() else 0


# ----------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, a_mn: bool = False, b_mn: bool = False,
         accumulate: bool = False, alpha: float = 1.0, out_dtype: torch.dtype | None = None, max_ctas: int = 0) -> torch.Tensor:
    """``out[M,N] (+)= alpha * A B^T`` with A given as [M,K] (or [K,M] when ``a_mn``) and B as [N,K] (or [K,N])."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype or a.dtype)
    if use_native(a, b) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16:
        a = a if a.stride(-1) == 1 else a.contiguous()
        b = b if b.stride(-1) == 1 else b.contiguous()
        ok = a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
        if ok:
            native().gemm(a, b, out, a_mn, b_mn, accumulate, alpha, status_word(a.device), max_ctas)
            return out
        note_fallback("gemm", "row stride not a multiple of 8 elements or base not 16-byte aligned", a, b)
    else:
        note_fallback("gemm", "operands are not both bf16", a, b)
    am = a.t() if a_mn else a
    bm = b if b_mn else b.t()
    res = (am.float() @ bm.float()) * alpha
    if accumulate:
        out.add_(res.to(out.dtype))
    else:
        out.copy_(res.to(out.dtype))
    return out


def _weight_grad_target(weight: torch.Tensor):
    """fp32 accumulation buffer attached by the sharded-training engine (None outside of it)."""
    return getattr(weight, "main_grad", None)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        with site("linear.fwd"):
            y = gemm(x2, weight)
        if bias is not None:
            y = y + bias
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            with site("linear.dgrad"):
                dx = gemm(dy2, weight, b_mn=True).view_as(x)
        if ctx.needs_input_grad[1]:
            target = _weight_grad_target(weight)
            with site("linear.wgrad"):
                if target is not None:
                    gemm(dy2, x2, target, a_mn=True, b_mn=True, accumulate=True)
                else:
                    dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if use_native(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _LinearFn.apply(x, weight, bias)
    note_fallback("linear", "input and weight are not both bf16 or the inner size is not a multiple of 8", x, weight)
    return F.linear(x, weight, bias)


# ----------------------------------------------------------------------------- RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual):
        xc = x.contiguous()
        with site("rmsnorm.fwd"):
            outs = native().rmsnorm_fwd(xc, None if residual is None else residual.contiguous(), weight, eps, True)
        if residual is None:
            y, rstd = outs
            h = xc
        else:
            y, rstd, h = outs
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_residual = residual is not None
        if residual is None:
            return y
        ctx.mark_non_differentiable()
        return y, h

    @staticmethod
    def backward(ctx, dy, dh_stream=None):
        h, weight, rstd = ctx.saved_tensors
        target = _weight_grad_target(weight)
        dw = None
        if target is not None:
            buf, acc = target, True
        else:
            buf, acc = torch.empty(weight.numel(), device=weight.device, dtype=torch.float32), False
        dres = None if dh_stream is None else dh_stream.contiguous()
        with site("rmsnorm.bwd"):
            dh = native().rmsnorm_bwd(dy.contiguous(), h, weight, rstd, dres, buf, acc)
        if target is None:
            dw = buf.to(weight.dtype)
        if ctx.has_residual:
            return dh, dw, None, dh
        return dh, dw, None, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, residual: torch.Tensor | None = None):
    """RMSNorm over the last dim. With ``residual`` returns ``(norm(x + residual), x + residual)``."""
    if weight is not None and use_native(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps, residual)
    note_fallback("rmsnorm", "no weight, mixed dtypes or a row length that is not a multiple of 8", x)
    h = x if residual is None else x + residual
    y = F.rms_norm(h, (h.shape[-1],), weight, eps)
    return y if residual is None else (y, h)


# ----------------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return native().swiglu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return native().swiglu_bwd(dy.contiguous(), x, False)[0]


def swiglu_packed(x: torch.Tensor) -> torch.Tensor:
    """``up * silu(gate)`` for ``x = [up | gate]`` along the last dim."""
    if use_native(x) and x.dtype == torch.bfloat16 and (x.shape[-1] // 2) % 8 == 0:
        return _SwiGLUFn.apply(x)
    note_fallback("swiglu", "intermediate size is not a multiple of 8", x)
    up, gate = x.chunk(2, dim=-1)
    return up * F.silu(gate)


# ----------------------------------------------------------------------------- RoPE on a fused projection
def rope_torch(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: torch.Tensor | None,
               groups: int, qpg: int, d: int, rd: int, inverse: bool = False) -> torch.Tensor:
    T = qkv.shape[0]
    v = qkv.reshape(T, groups, qpg + 2, d)
    pos = position_ids.long() if position_ids is not None else torch.arange(T, device=qkv.device)
    c = torch.cat([cos, cos], -1)[pos][:, None, None, :].to(torch.float32)
    s = torch.cat([sin, sin], -1)[pos][:, None, None, :].to(torch.float32)
    if inverse:
        s = -s
    rot = v[:, :, : qpg + 1, d - rd :].float()
    x1, x2 = rot.chunk(2, -1)
    rotated = rot * c + torch.cat([-x2, x1], -1) * s
    out = v.clone()
    out[:, :, : qpg + 1, d - rd :] = rotated.to(qkv.dtype)
    return out.reshape(T, -1)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, position_ids, groups, qpg, d, rd):
        ctx.save_for_backward(cos, sin, position_ids)
        ctx.meta = (groups, qpg, d, rd)
        out = qkv.contiguous().clone() if qkv.requires_grad else qkv.contiguous()
        native().rope_(out, cos, sin, position_ids, groups, qpg, d, rd, False)
        return out

    @staticmethod
    def backward(ctx, dout):
        cos, sin, position_ids = ctx.saved_tensors
        groups, qpg, d, rd = ctx.meta
        dq = dout.contiguous().clone()
        native().rope_(dq, cos, sin, position_ids, groups, qpg, d, rd, True)
        return dq, None, None, None, None, None, None, None


def rope_fused_qkv(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: torch.Tensor | None,
                   groups: int, qpg: int, d: int, rd: int) -> torch.Tensor:
    """Rotate the query and key heads of a fused ``[T, groups * (qpg + 2) * d]`` projection (half-rotation form)."""
    if use_native(qkv) and qkv.dtype == torch.bfloat16 and rd % 16 == 0 and cos.dtype == torch.float32:
        pid = None if position_ids is None else position_ids.to(torch.int32).contiguous()
        return _RopeFn.apply(qkv, cos.contiguous(), sin.contiguous(), pid, groups, qpg, d, rd)
    note_fallback("rope", "rotary dimension is not a multiple of 16 or the tables are not fp32", qkv)
    return rope_torch(qkv, cos, sin, position_ids, groups, qpg, d, rd)


# ----------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight, ids, scale):
        ctx.save_for_backward(ids)
        ctx.weight = weight
        ctx.scale = scale
        return native().embedding_fwd(weight, ids.contiguous(), scale)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        weight = ctx.weight
        target = _weight_grad_target(weight)
        if target is not None:
            native().embedding_bwd(dy.contiguous(), ids.contiguous(), target.view(weight.shape), ctx.scale)
            return None, None, None
        dw = torch.zeros(weight.shape, device=weight.device, dtype=torch.float32)
        native().embedding_bwd(dy.contiguous(), ids.contiguous(), dw, ctx.scale)
        return dw.to(weight.dtype), None, None


def embedding(weight: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if use_native(weight) and weight.dtype == torch.bfloat16 and ids.is_cuda and weight.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(weight, ids.long(), float(scale))
    note_fallback("embedding", "hidden size is not a multiple of 8 or the ids are not on the device", weight)
    out = F.embedding(ids, weight)
    return out if scale == 1.0 else out * scale


# ----------------------------------------------------------------------------- fused linear + cross entropy
def _flce_chunk_rows(T: int, V: int) -> int:
    # One pass over the fp32 weight-gradient accumulator per chunk is the dominant extra traffic of this op, so chunks
    # are as large as a ~2.2 GB transient bf16 logits buffer allows (the whole micro-batch for 8k tokens x 128k vocab).
    rows = max(256, (1100 * 1024 * 1024) // max(V, 1))
    rows = (rows // 128) * 128 or 128
    return min(T, rows)


class _FusedLinearCrossEntropyFn(torch.autograd.Function):
    """loss = sum_t CE(logit_scale * x_t W^T, label_t) without keeping [T, V] logits.

    Forward walks token chunks: logits chunk (tcgen05 GEMM) -> in-place softmax gradient (CE kernel) -> dX chunk and
    dW accumulation (two more GEMMs), so backward only scales what forward produced.
    """

    @staticmethod
    def forward(ctx, x, weight, labels, logit_scale, ignore_index, grad_scale):
        T, H = x.shape
        V = weight.shape[0]
        trusted = grad_scale is not None
        gs = float(grad_scale) if trusted else 1.0
        C = native()
        need_dx = x.requires_grad
        need_dw = weight.requires_grad
        target = _weight_grad_target(weight) if need_dw else None
        dx = torch.empty_like(x) if need_dx else None
        dw = None
        if need_dw and target is None:
            dw = torch.zeros(V, H, device=x.device, dtype=torch.float32)
        dw_buf = target.view(V, H) if target is not None else dw
        rows = _flce_chunk_rows(T, V)
        logits = torch.empty(rows, V, device=x.device, dtype=torch.bfloat16)
        loss_rows = torch.empty(T, device=x.device, dtype=torch.float32)
        st = status_word(x.device)
        for start in range(0, T, rows):
            n = min(rows, T - start)
            xc = x[start : start + n]
            lg = logits[:n]
            with site("loss.lm_head.logits"):
                C.gemm(xc, weight, lg, False, False, False, 1.0, st, 0)
            with site("loss.cross_entropy"):
                loss_rows[start : start + n] = C.cross_entropy_(lg, labels[start : start + n], logit_scale, gs, ignore_index, need_dx or need_dw)
            if need_dx:
                with site("loss.lm_head.dgrad"):
                    C.gemm(lg, weight, dx[start : start + n], False, True, False, 1.0, st, 0)
            if need_dw:
                with site("loss.lm_head.wgrad"):
                    C.gemm(lg, xc, dw_buf, True, True, True, 1.0, st, 0)
        ctx.dx = dx
        ctx.dw = dw
        ctx.accumulated_in_place = target is not None
        ctx.trusted = trusted
        ctx.grad_scale = gs
        ctx.status = st
        ctx.weight_dtype = weight.dtype
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.dx, ctx.dw
        ctx.dx = ctx.dw = None
        if not ctx.trusted:
            if dx is not None:
                dx = dx * dloss.to(dx.dtype)
            if dw is not None:
                dw = dw * dloss
        if dw is not None:
            dw = dw.to(ctx.weight_dtype)
        # `trusted`: the caller passed the upstream gradient of the summed loss as `grad_scale`, so the stored
        # gradients (and whatever was accumulated into an engine-owned fp32 buffer) are already final. The claim is
        # checked on the device, without a host sync: an upstream gradient that differs from the promised scale raises
        # the status word, which `check_status()` turns into an error at the next log / save point.
        if ctx.trusted:
            promised = ctx.grad_scale
            wrong = (dloss.detach().float().reshape(()) - promised).abs() > 1e-4 * abs(promised) + 1e-30
            ctx.status.copy_(torch.where(wrong & (ctx.status == 0), torch.full_like(ctx.status, STATUS_GRAD_SCALE_MISMATCH), ctx.status))
        return dx, dw, None, None, None, None


def fused_linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, *, logit_scale: float = 1.0,
                               ignore_index: int = -100, reduction: str = "sum", grad_scale_hint: float | None = None) -> torch.Tensor:
    """Cross entropy of ``logit_scale * (x @ weight.T)`` against ``labels`` (sum or mean over non-ignored rows)."""
    x2 = x.reshape(-1, x.shape[-1])
    lab = labels.reshape(-1)
    if use_native(x2, weight) and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x2.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0:
        loss = _FusedLinearCrossEntropyFn.apply(x2.contiguous(), weight, lab.long().contiguous(), float(logit_scale), ignore_index, grad_scale_hint)
    else:
        note_fallback("fused_linear_cross_entropy", "mixed dtypes or sizes that are not multiples of 8", x2, weight)
        logits = F.linear(x2, weight).float() * logit_scale
        loss = F.cross_entropy(logits, lab.long(), ignore_index=ignore_index, reduction="sum")
    if reduction == "mean":
        loss = loss / (lab != ignore_index).sum().clamp(min=1)
    return loss


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, *, ignore_index: int = -100, reduction: str = "sum") -> torch.Tensor:
    """fp32 cross entropy on materialised logits."""
    loss = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1).long(), ignore_index=ignore_index, reduction=reduction)
    return loss

"""Tensor-parallel communication as explicit autograd functions over the tensor-parallel process group.

The reference expresses these as DTensor redistributions (lm_engine/dtensors.py:12-86 and
lm_engine/hf_models/modeling_utils_TP/linear.py:107-113, 170-174 there); here every crossing of a layout boundary is
one function whose backward is the transposed collective:

====================  =========================  =========================
function              forward                    backward
====================  =========================  =========================
``copy_to_tp``        identity                   all-reduce
``reduce_from_tp``    all-reduce                 identity
``gather_tokens``     all-gather (token dim)     reduce-scatter
``scatter_tokens``    reduce-scatter (token dim) all-gather
``gather_features``   all-gather (last dim)      slice
====================  =========================  =========================

With sequence parallelism the regions between the linears (norms, dropout, residual adds) hold ``tokens / tp`` rows, a
column-parallel linear gathers its input and a row-parallel linear reduce-scatters its output; without it the
activations are replicated and the pair is identity / all-reduce. On B200 with bf16 activations the gather + GEMM and
GEMM + reduce-scatter pairs run as single kernels over peer memory (:mod:`lm_engine.parallel.fused_tp`).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..utils import ProcessGroupManager


def tp_world() -> int:
    return ProcessGroupManager.get_tensor_parallel_world_size() if ProcessGroupManager.is_initialized() else 1


def tp_rank() -> int:
    return ProcessGroupManager.get_tensor_parallel_rank() if ProcessGroupManager.is_initialized() else 0


def tp_group():
    return ProcessGroupManager.get_tensor_parallel_group()


# ----------------------------------------------------------------------------------------------------------------------
# raw collectives that work on gloo and NCCL alike
def _all_gather(x: torch.Tensor, dim: int) -> torch.Tensor:
    world = tp_world()
    if world == 1:
        return x
    x = x.contiguous()
    if x.is_cuda and dim == 0:
        out = x.new_empty((x.shape[0] * world, *x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=tp_group())
        return out
    pieces = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(pieces, x, group=tp_group())
    return torch.cat(pieces, dim=dim)


def _reduce_scatter(x: torch.Tensor, dim: int) -> torch.Tensor:
    world = tp_world()
    if world == 1:
        return x
    x = x.contiguous()
    if x.is_cuda and dim == 0:
        out = x.new_empty((x.shape[0] // world, *x.shape[1:]))
        dist.reduce_scatter_tensor(out, x, group=tp_group())
        return out
    if x.is_cuda:
        pieces = [p.contiguous() for p in x.chunk(world, dim=dim)]
        out = torch.empty_like(pieces[0])
        dist.reduce_scatter(out, pieces, group=tp_group())
        return out
    total = x.clone()
    dist.all_reduce(total, group=tp_group())  # gloo has no reduce-scatter
    return total.chunk(world, dim=dim)[tp_rank()].contiguous()


def _all_reduce(x: torch.Tensor) -> torch.Tensor:
    if tp_world() == 1:
        return x
    x = x.contiguous().clone()
    dist.all_reduce(x, group=tp_group())
    return x


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g)


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _all_reduce(x)

    @staticmethod
    def backward(ctx, g):
        return g


class _GatherTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _all_gather(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g, ctx.dim), None


class _ScatterTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _reduce_scatter(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _all_gather(g, ctx.dim), None


class _GatherFeatures(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _all_gather(x, x.dim() - 1)

    @staticmethod
    def backward(ctx, g):
        return g.chunk(tp_world(), dim=-1)[tp_rank()].contiguous()


class _SliceTokens(torch.autograd.Function):
    """Replicated -> sequence-sharded without communication (backward gathers)."""

    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return x.chunk(tp_world(), dim=dim)[tp_rank()].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather(g, ctx.dim), None


def copy_to_tp(x: torch.Tensor) -> torch.Tensor:
    return x if tp_world() == 1 else _Copy.apply(x)


def reduce_from_tp(x: torch.Tensor) -> torch.Tensor:
    return x if tp_world() == 1 else _Reduce.apply(x)


def gather_tokens(x: torch.Tensor, dim: int) -> torch.Tensor:
    return x if tp_world() == 1 else _GatherTokens.apply(x, dim)


def scatter_tokens(x: torch.Tensor, dim: int) -> torch.Tensor:
    return x if tp_world() == 1 else _ScatterTokens.apply(x, dim)


def gather_features(x: torch.Tensor) -> torch.Tensor:
    return x if tp_world() == 1 else _GatherFeatures.apply(x)


def slice_tokens(x: torch.Tensor, dim: int) -> torch.Tensor:
    return x if tp_world() == 1 else _SliceTokens.apply(x, dim)


def token_dim(x: torch.Tensor) -> int:
    """Packed activations are ``[tokens, hidden]`` (dim 0); padded ones ``[batch, sequence, hidden]`` (dim 1)."""
    return 0 if x.dim() == 2 else 1


# ----------------------------------------------------------------------------------------------------------------------
def column_parallel_input(x: torch.Tensor, sequence_parallel: bool) -> torch.Tensor:
    return gather_tokens(x, token_dim(x)) if sequence_parallel else copy_to_tp(x)


def row_parallel_output(y: torch.Tensor, sequence_parallel: bool) -> torch.Tensor:
    return scatter_tokens(y, token_dim(y)) if sequence_parallel else reduce_from_tp(y)


# ----------------------------------------------------------------------------------------------------------------------
# reductions that run under the next piece of compute (ladder residual)
class _StartReduction(torch.autograd.Function):
    """Starts the all-reduce / reduce-scatter of a row-parallel output and returns at once. The result must not be read
    before :func:`finish_reduction` has been applied to it. Backward is the transposed collective of the synchronous
    functions (identity / all-gather), run in place."""

    @staticmethod
    def forward(ctx, y, sequence_parallel):
        ctx.sequence_parallel = sequence_parallel
        ctx.dim = token_dim(y)
        world = tp_world()
        y = y.contiguous()
        ctx.sliced_later = False
        if not sequence_parallel:
            out = y.clone()
            work = dist.all_reduce(out, group=tp_group(), async_op=True)
        elif y.is_cuda and ctx.dim == 0:
            out = y.new_empty((y.shape[0] // world, *y.shape[1:]))
            work = dist.reduce_scatter_tensor(out, y, group=tp_group(), async_op=True)
            out._reduction_input = y  # the input must stay alive until the collective has read it
        else:
            total = y.clone()
            work = dist.all_reduce(total, group=tp_group(), async_op=True)  # gloo has no reduce-scatter
            out = total
            out._slice = (ctx.dim, world, tp_rank())
            ctx.sliced_later = True
        out._pending_reduction = work
        return out

    @staticmethod
    def backward(ctx, g):
        if ctx.sliced_later:
            return _all_reduce(g), None  # g holds this rank's slice and zeros elsewhere: the sum over ranks is the gather
        return (_all_gather(g, ctx.dim) if ctx.sequence_parallel else g), None


class _FinishReduction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        work = getattr(x, "_pending_reduction", None)
        if work is not None:
            work.wait()
            x._pending_reduction = None
        piece = getattr(x, "_slice", None)
        ctx.piece = piece
        if piece is not None:
            dim, world, rank = piece
            return x.chunk(world, dim=dim)[rank].contiguous()
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.piece is not None:
            dim, world, rank = ctx.piece
            shape = list(g.shape)
            shape[dim] *= world
            full = g.new_zeros(shape)
            full.narrow(dim, rank * g.shape[dim], g.shape[dim]).copy_(g)
            return full
        return g


def row_parallel_output_async(y: torch.Tensor, sequence_parallel: bool) -> torch.Tensor:
    """Like :func:`row_parallel_output`, but only STARTS the collective (on the communication library's own stream):
    the caller goes on with independent work and applies :func:`finish_reduction` where the value is needed."""
    if tp_world() == 1:
        return y
    return _StartReduction.apply(y, sequence_parallel)


def finish_reduction(x: torch.Tensor | None) -> torch.Tensor | None:
    """Wait for a reduction started by :func:`row_parallel_output_async` (no-op for anything else)."""
    if x is None or not (hasattr(x, "_pending_reduction") or hasattr(x, "_slice")):
        return x
    return _FinishReduction.apply(x)


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Cross entropy over logits whose vocabulary dimension is split across the group: three small all-reduces (row
    maximum, sum of exponentials, target logit) instead of gathering ``[tokens, vocab]``."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, ignore_index):
        x = logits.float()
        local_max = x.max(dim=-1).values
        if tp_world() > 1:
            dist.all_reduce(local_max, op=dist.ReduceOp.MAX, group=tp_group())
        x = x - local_max.unsqueeze(-1)
        exp = x.exp()
        denom = exp.sum(dim=-1)
        local = labels - vocab_start
        mine = (local >= 0) & (local < x.shape[-1]) & (labels != ignore_index)
        safe = local.clamp(0, x.shape[-1] - 1)
        target = x.gather(-1, safe.unsqueeze(-1)).squeeze(-1) * mine
        if tp_world() > 1:
            dist.all_reduce(denom, group=tp_group())
            dist.all_reduce(target, group=tp_group())
        valid = labels != ignore_index
        loss = (denom.log() - target) * valid
        ctx.save_for_backward(exp / denom.unsqueeze(-1), safe, mine, valid)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        softmax, safe, mine, valid = ctx.saved_tensors
        grad = softmax.clone()
        grad.scatter_add_(-1, safe.unsqueeze(-1), -mine.unsqueeze(-1).to(grad.dtype))
        grad = grad * (grad_loss * valid).unsqueeze(-1)
        return grad.to(ctx.dtype), None, None, None


def combine_shard_statistics(stats: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``stats``: ``[ranks, T, 3]`` = every rank's (row maximum, sum of exponentials relative to it, target logit or 0).
    Returns ``(log-sum-exp over the whole vocabulary, target logit)`` per row."""
    top = stats[:, :, 0].max(dim=0).values
    total = (stats[:, :, 1] * torch.exp(stats[:, :, 0] - top)).sum(dim=0)
    return top + torch.log(total), stats[:, :, 2].sum(dim=0)


class _VocabParallelCrossEntropyNative(torch.autograd.Function):
    """The same loss with this library's kernels: one pass over the rank's logits for the three row statistics, ONE
    all-gather of ``[T, 3]`` floats instead of three all-reduces, and in backward one pass that writes the rank's
    slice of the gradient from the saved bf16 logits (no fp32 softmax is kept)."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, ignore_index):
        from .. import ops

        C = ops.native()
        stats = C.ce_shard_stats(logits, labels, vocab_start, ignore_index)
        world = tp_world()
        if world > 1:
            gathered = stats.new_empty((world, *stats.shape))
            dist.all_gather_into_tensor(gathered, stats, group=tp_group())
        else:
            gathered = stats.unsqueeze(0)
        lse, target = combine_shard_statistics(gathered)
        valid = labels != ignore_index
        ctx.save_for_backward(logits, labels, lse)
        ctx.meta = (vocab_start, ignore_index)
        return (lse - target) * valid

    @staticmethod
    def backward(ctx, grad_loss):
        from .. import ops

        logits, labels, lse = ctx.saved_tensors
        vocab_start, ignore_index = ctx.meta
        grad = ops.native().ce_shard_grad(logits, labels, lse, grad_loss.float().contiguous(), vocab_start, ignore_index)
        return grad, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, reduction: str = "mean", ignore_index: int = -100,
                                 vocab_start: int | None = None) -> torch.Tensor:
    """``logits``: ``[..., vocab / tp]`` (this rank's slice, starting at ``vocab_start``), ``labels``: replicated."""
    from .. import ops

    if vocab_start is None:
        vocab_start = tp_rank() * logits.shape[-1]
    flat = logits.reshape(-1, logits.shape[-1])
    labels = labels.reshape(-1)
    if flat.is_cuda and flat.dtype == torch.bfloat16 and ops.native_available() and hasattr(ops.native(), "ce_shard_stats"):
        per_token = _VocabParallelCrossEntropyNative.apply(flat.contiguous(), labels.long().contiguous(), vocab_start, ignore_index)
    else:
        ops.note_fallback("vocab_parallel_cross_entropy", "logits are not bf16", flat)
        per_token = _VocabParallelCrossEntropy.apply(flat, labels, vocab_start, ignore_index)
    total = per_token.sum()
    if reduction == "sum":
        return total
    return total / (labels != ignore_index).sum().clamp(min=1)


def vocab_parallel_embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int) -> torch.Tensor:
    """Rows of a vocabulary-sharded table; ids owned by other ranks give zeros (the caller reduces over the group)."""
    local = ids - vocab_start
    mine = (local >= 0) & (local < weight.shape[0])
    out = F.embedding(local.clamp(0, weight.shape[0] - 1), weight)
    return out * mine.unsqueeze(-1).to(out.dtype)

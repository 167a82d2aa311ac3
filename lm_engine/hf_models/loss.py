"""Language-modelling loss and the per-forward auxiliary-loss accumulator.

Parity: lm_engine/hf_models/loss.py:23-116. ``get_autoregressive_language_modeling_loss`` optionally shifts
logits/labels, masks the last token of every packed document when shifting, and picks between the fused
linear+cross-entropy kernel (no ``[T, V]`` logits are kept), a cross-entropy on given logits, and a vocab-parallel
variant under tensor parallelism.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..enums import Kernel
from ..kernels import is_kernel_allowed

_AUX_LOSS: torch.Tensor | float = 0
# Router statistics of the MoE layers of the current forward pass, turned into their auxiliary losses when the loss is
# asked for: (probability mass per expert [E] (differentiable), tokens per expert [E], z term, dtype of the logits).
_ROUTER_STATISTICS: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.dtype]] = []


def clear_aux_loss() -> None:
    global _AUX_LOSS
    _AUX_LOSS = 0
    _ROUTER_STATISTICS.clear()


def add_aux_loss(aux_loss: torch.Tensor | float) -> None:
    global _AUX_LOSS
    _AUX_LOSS = _AUX_LOSS + aux_loss


def add_router_statistics(probability_mass: torch.Tensor, tokens_per_expert: torch.Tensor, z_term: torch.Tensor,
                          dtype: torch.dtype) -> None:
    """One MoE layer's share of the load-balancing loss, left unfinished: the token counts of all layers are summed over
    the data-parallel group by ONE collective in `get_aux_loss` instead of one per layer (the counts carry no gradient,
    so the value and the gradients are those of the per-layer formulation,
    lm_engine/hf_models/modeling_utils/mlp_blocks/moe.py:259-290 in the reference)."""
    _ROUTER_STATISTICS.append((probability_mass, tokens_per_expert, z_term, dtype))


def _finish_router_statistics() -> torch.Tensor:
    from ..utils import ProcessGroupManager

    probability_mass = torch.stack([p for p, _, _, _ in _ROUTER_STATISTICS])           # [layers, experts]
    tokens = torch.stack([f for _, f, _, _ in _ROUTER_STATISTICS]).float()             # [layers, experts]
    z = torch.stack([z for _, _, z, _ in _ROUTER_STATISTICS])                          # [layers]
    dtype = _ROUTER_STATISTICS[0][3]
    _ROUTER_STATISTICS.clear()
    if ProcessGroupManager.is_initialized() and ProcessGroupManager.get_data_parallel_world_size() > 1:
        dist.all_reduce(tokens, group=ProcessGroupManager.get_data_parallel_group())
    num_experts = probability_mass.shape[-1]
    balance = num_experts * (F.normalize(probability_mass, p=1, dim=-1) * F.normalize(tokens, p=1, dim=-1)).sum(-1)
    return (balance + 0.1 * z).to(dtype).sum()  # rounded per layer, as if every layer had added its own term


def get_aux_loss() -> torch.Tensor | float:
    global _AUX_LOSS
    if _ROUTER_STATISTICS:
        _AUX_LOSS = _AUX_LOSS + _finish_router_statistics()
    return _AUX_LOSS


def is_aux_loss_zero(aux_loss: torch.Tensor | float) -> bool:
    return isinstance(aux_loss, (int, float)) and aux_loss == 0


def get_autoregressive_language_modeling_loss(
    lm_logits: torch.Tensor | None,
    labels: torch.Tensor,
    hidden_states: torch.Tensor | None = None,
    vocab_weight: torch.Tensor | None = None,
    cu_seqlens: torch.Tensor | None = None,
    use_padding_free_transformer: bool = False,
    reduction: str = "mean",
    shift_logits_and_labels: bool = True,
    tensor_parallel_enabled: bool = False,
    logit_scale: float = 1.0,
    grad_scale_hint: float | None = None,
) -> torch.Tensor:
    """Next-token cross entropy (ignored label = -100).

    Either ``lm_logits`` or (``hidden_states``, ``vocab_weight``) must be given; the latter selects the fused
    linear + cross-entropy path, where ``logit_scale`` (``1 / m_width``) is applied inside the kernel.
    """
    if reduction not in ("sum", "mean"):
        raise ValueError(f"unexpected reduction ({reduction})")
    fused = lm_logits is None
    if fused and tensor_parallel_enabled:
        # the LM head is split over the vocabulary under tensor parallelism: a softmax over this rank's slice alone,
        # with labels that are not offset, would be silently wrong (the reference asserts the same)
        raise ValueError("fused linear + cross entropy cannot be combined with tensor parallelism; pass the "
                         "vocabulary-parallel logits instead")
    x = hidden_states if fused else lm_logits

    if use_padding_free_transformer:
        if shift_logits_and_labels:
            if cu_seqlens is None:
                raise ValueError("cu_seqlens is needed to shift labels of packed documents")
            # token t predicts t + 1; the last token of every document predicts nothing
            labels = torch.cat([labels[1:], labels.new_full((1,), -100)])
            labels[cu_seqlens[1:] - 1] = -100
    elif shift_logits_and_labels:
        x = x[..., :-1, :]
        labels = labels[..., 1:]

    if tensor_parallel_enabled and not fused:
        from ..parallel.tensor_parallel import vocab_parallel_cross_entropy

        return vocab_parallel_cross_entropy(x, labels, reduction=reduction)

    if fused:
        return ops.fused_linear_cross_entropy(x, vocab_weight, labels, logit_scale=logit_scale, reduction=reduction,
                                              grad_scale_hint=grad_scale_hint)
    if logit_scale != 1.0:
        x = x * logit_scale
    return ops.cross_entropy(x, labels, reduction=reduction)

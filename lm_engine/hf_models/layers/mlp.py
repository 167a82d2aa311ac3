"""Feed-forward blocks: dense MLP and sparse mixture of experts.

Parity: lm_engine/hf_models/modeling_utils/mlp_blocks/{mlp.py:15-73, moe.py:47-384}. MoE routing: logits ->
top-k (max for k = 1) -> softmax over the k selected logits in fp32; no capacity limit, no token dropping.
Expert weights are ``c_fc.weight [E, I or 2I, H]`` and ``c_proj.weight [E, H, I]``. The auxiliary loss is
``E * sum(normalize(sum probs) * normalize(freq)) + 0.1 * mean(logsumexp(logits)^2)`` with ``freq`` summed over the
data parallel group, accumulated into a per-forward global (see :mod:`lm_engine.hf_models.loss`).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...enums import Kernel
from ...kernels import is_kernel_allowed
from ...utils import ProcessGroupManager
from ..loss import add_aux_loss, add_router_statistics
from ..parameter import mark_parameter_as_mup_learning_rate, mark_parameter_as_no_weight_decay
from .activations import get_activation_function, is_glu
from .basic import ParameterizedLinear, init_zeros_


def _std(initializer_range: float, init_method: str, m_width: float | None, depth_scale: int | None = None) -> float:
    std = initializer_range
    if depth_scale is not None:
        std /= math.sqrt(2 * depth_scale)
    if init_method == "mup":
        std /= math.sqrt(m_width)
    return std


def interleave_up_gate_tensor_for_mlp(up_weight: torch.Tensor, gate_weight: torch.Tensor) -> torch.Tensor:
    """The fused ``c_fc`` of a gated MLP: rows ``[up ; gate]``."""
    return torch.cat((up_weight, gate_weight), dim=0)


def split_up_gate_tensor_for_mlp(c_fc_weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`interleave_up_gate_tensor_for_mlp`."""
    half = c_fc_weight.shape[0] // 2
    return c_fc_weight[:half], c_fc_weight[half:]


class MLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, activation_function: str, add_bias: bool,
                 dropout: float, init_method: str, initializer_range: float, m_width: float | None,
                 num_layers: int) -> None:
        super().__init__()
        self.is_glu = is_glu(activation_function)
        self.c_fc = ParameterizedLinear(hidden_size, 2 * intermediate_size if self.is_glu else intermediate_size,
                                        bias=add_bias, std=_std(initializer_range, init_method, m_width))
        self.act = get_activation_function(activation_function)
        self.c_proj = ParameterizedLinear(intermediate_size, hidden_size, bias=add_bias,
                                          std=_std(initializer_range, init_method, m_width, num_layers))
        self.dropout = nn.Identity() if dropout == 0 else nn.Dropout(dropout)
        mark_parameter_as_mup_learning_rate(self.c_fc.weight)
        mark_parameter_as_mup_learning_rate(self.c_proj.weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dropout(self.c_proj(self.act(self.c_fc(x))))


class ParameterizedExperts(nn.Module):
    """A bank of ``num_experts`` linear maps stored as one ``[E, out, in]`` tensor."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = False,
                 std: float | None = None) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.std = std
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if add_bias else None
        mark_parameter_as_no_weight_decay(self.bias)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0.0, std=self.std if self.std is not None else 0.02)
        init_zeros_(self.bias)

    def forward_grouped(self, x: torch.Tensor, tokens_per_expert: list[int]) -> torch.Tensor:
        """``x`` holds the rows of expert 0, then expert 1, ...; one dense product per non-empty expert."""
        outs = []
        start = 0
        for e, n in enumerate(tokens_per_expert):
            if n == 0:
                continue
            b = None if self.bias is None else self.bias[e]
            outs.append(F.linear(x[start : start + n], self.weight[e], b))
            start += n
        if not outs:
            return x.new_zeros(0, self.out_features)
        return torch.cat(outs, dim=0)

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.in_features}, out_features={self.out_features}"


class ExpertParallelExperts(ParameterizedExperts):
    """The ``num_experts / ep`` experts of this rank of the expert-parallel group. Initialisation draws the whole bank
    and keeps this rank's experts, so the group starts from the weights a single device would have."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = False, std: float | None = None) -> None:
        self.ep_world = ProcessGroupManager.get_expert_parallel_world_size()
        self.ep_rank = ProcessGroupManager.get_expert_parallel_rank()
        self.num_global_experts = num_experts
        if num_experts % self.ep_world != 0:
            raise ValueError("the number of experts must be divisible by the expert parallel size")
        super().__init__(num_experts // self.ep_world, in_features, out_features, add_bias=add_bias, std=std)
        for p in self.parameters():
            p._expert_parallel = True

    @torch.no_grad()
    def reset_parameters(self) -> None:
        from .basic import loaded_from_checkpoint

        if not loaded_from_checkpoint(self.weight):
            full = torch.empty(self.num_global_experts, *self.weight.shape[1:], dtype=torch.float32, device=self.weight.device)
            full.normal_(mean=0.0, std=self.std if self.std is not None else 0.02)
            self.weight.copy_(full.chunk(self.ep_world)[self.ep_rank])
        init_zeros_(self.bias)


def _expert_parallel_world() -> int:
    return ProcessGroupManager.get_expert_parallel_world_size() if ProcessGroupManager.is_initialized() else 1


class MoE(nn.Module):
    linear_class = ParameterizedExperts

    def __init__(self, hidden_size: int, intermediate_size: int, shared_intermediate_size: int | None,
                 num_experts: int, num_experts_per_tok: int, activation_function: str, add_bias: bool,
                 dropout: float, init_method: str, initializer_range: float, m_width: float | None,
                 num_layers: int, use_padding_free_transformer: bool) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.shared_intermediate_size = shared_intermediate_size
        self.use_padding_free_transformer = use_padding_free_transformer
        self.is_glu = is_glu(activation_function)
        self.activation_function = activation_function
        width = 2 if self.is_glu else 1

        self.gate = ParameterizedLinear(hidden_size, num_experts, bias=False, std=_std(initializer_range, init_method, m_width))
        self.expert_parallel = _expert_parallel_world() > 1
        bank = ExpertParallelExperts if self.expert_parallel else ParameterizedExperts
        self.c_fc = bank(num_experts, hidden_size, width * intermediate_size, add_bias=add_bias,
                         std=_std(initializer_range, init_method, m_width))
        if shared_intermediate_size is not None:
            self.c_fc_shared = ParameterizedLinear(hidden_size, width * shared_intermediate_size, bias=add_bias,
                                                   std=_std(initializer_range, init_method, m_width))
        self.act = get_activation_function(activation_function)
        self.c_proj = bank(num_experts, intermediate_size, hidden_size, add_bias=add_bias,
                           std=_std(initializer_range, init_method, m_width, num_layers))
        if shared_intermediate_size is not None:
            self.c_proj_shared = ParameterizedLinear(shared_intermediate_size, hidden_size, bias=add_bias,
                                                     std=_std(initializer_range, init_method, m_width, num_layers))
        self.dropout = nn.Identity() if dropout == 0 else nn.Dropout(dropout)

        for module in (self.gate, self.c_fc, self.c_proj):
            mark_parameter_as_mup_learning_rate(module.weight)
        if shared_intermediate_size is not None:
            mark_parameter_as_mup_learning_rate(self.c_fc_shared.weight)
            mark_parameter_as_mup_learning_rate(self.c_proj_shared.weight)

    # ------------------------------------------------------------------ routing
    def route(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        logits = self.gate(x)
        if x.is_cuda and logits.dim() == 2 and is_kernel_allowed(Kernel.scattermoe):
            from ...ops.sequence import topk_route

            # one kernel: top-k, softmax of the selected logits and (while training) the tokens per expert
            weights, experts, counts = topk_route(logits, self.top_k, want_counts=self.training)
            self._tokens_per_expert = counts
            return logits, weights.type_as(x), experts
        if self.top_k == 1:
            top_logits, experts = logits.max(dim=-1, keepdim=True)
        else:
            top_logits, experts = logits.topk(self.top_k, dim=-1)
        weights = F.softmax(top_logits.float(), dim=-1).type_as(x)
        self._tokens_per_expert = None
        return logits, weights, experts

    # ------------------------------------------------------------------ experts
    def _experts_torch(self, x: torch.Tensor, weights: torch.Tensor, experts: torch.Tensor) -> torch.Tensor:
        flat = experts.flatten()
        counts = torch.bincount(flat, minlength=self.num_experts).tolist()
        order = flat.argsort(stable=True)
        token_of_row = order // self.top_k
        h = self.c_fc.forward_grouped(x[token_of_row], counts)
        h = self.act(h)
        h = self.c_proj.forward_grouped(h, counts)
        h = h * weights.flatten()[order].unsqueeze(-1)
        return torch.zeros_like(x).index_add(0, token_of_row, h)

    def _experts_native(self, x: torch.Tensor, weights: torch.Tensor, experts: torch.Tensor) -> torch.Tensor:
        from ...ops.moe import scattered_experts_mlp

        return scattered_experts_mlp(x, self.c_fc.weight, self.c_proj.weight, weights, experts, self.num_experts,
                                     self.top_k, self.activation_function)

    def experts(self, x: torch.Tensor, weights: torch.Tensor, selected: torch.Tensor) -> torch.Tensor:
        if self.expert_parallel:
            from ...parallel.expert_parallel import expert_parallel_mlp

            return expert_parallel_mlp(x, self.c_fc.weight, self.c_proj.weight, self.c_fc.bias, self.c_proj.bias, weights, selected,
                                       self.num_experts, self.top_k, self.activation_function, self.act)
        if is_kernel_allowed(Kernel.scattermoe) and self.c_fc.bias is None:
            from ...ops.moe import native_moe_ok

            if native_moe_ok(x, self.activation_function):
                return self._experts_native(x, weights, selected)
        return self._experts_torch(x, weights, selected)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        logits, weights, selected = self.route(x)
        out = self.experts(x, weights, selected)
        if self.shared_intermediate_size is not None:
            out = out + self.c_proj_shared(self.act(self.c_fc_shared(x)))
        out = self.dropout(out.reshape(shape))
        if self.training:
            self._router_statistics(logits, selected)
        return out

    def _router_statistics(self, logits: torch.Tensor, selected: torch.Tensor) -> None:
        """Load-balancing and z loss of this layer, handed to the loss module unfinished (see `add_router_statistics`)."""
        logits = logits.reshape(-1, logits.shape[-1])
        probs = torch.softmax(logits, dim=-1)
        counts = getattr(self, "_tokens_per_expert", None)
        self._tokens_per_expert = None
        if counts is None:
            # no host synchronisation (bincount needs one to size its output)
            counts = torch.zeros(self.num_experts, device=logits.device, dtype=torch.float32)
            counts.index_add_(0, selected.flatten(), torch.ones(selected.numel(), device=logits.device, dtype=torch.float32))
        z = (torch.logsumexp(logits, dim=-1) ** 2).mean()
        add_router_statistics(probs.sum(0), counts.float(), z, logits.dtype)

    def get_num_active_parameters(self) -> int:
        total = sum(p.numel() for p in self.parameters())
        for bank in (self.c_fc, self.c_proj):
            for p in bank.parameters():
                total -= p.numel()
                total += (p.numel() * self.top_k) // self.num_experts
        return total

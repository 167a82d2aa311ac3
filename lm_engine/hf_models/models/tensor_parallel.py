"""Tensor-parallel (and pipeline-stage) variants of the dense model family.

Parity: lm_engine/hf_models/modeling_utils_TP/* (layers), lm_engine/hf_models/mixins/dense_TP/{base,layer,main}.py
(model), lm_engine/hf_models/models/{gpt_base_TP,ladder_residual_TP}. The reference makes every parameter a DTensor and
lets redistributions produce the collectives; here each rank holds plain local tensors and the layers call the explicit
collectives of :mod:`lm_engine.parallel.tensor_parallel`.

Layouts (tp = tensor-parallel size, r = rank):
  * column-parallel linear: rows ``[r * out / tp, (r + 1) * out / tp)``; a gated ``c_fc`` keeps ``[up_r ; gate_r]`` so
    that the local activation splits the same way; the fused ``c_attn`` is sharded by whole key/value groups.
  * row-parallel linear: columns ``[r * in / tp, ...)``; the bias is replicated and added after the reduction.
  * embedding / LM head: vocabulary rows, the vocabulary padded to a multiple of 64.
  * norms, router, row-parallel biases and the multi-query ``kv_attn`` are replicated. Their gradients are
    partial sums whenever their input or their consumers are sharded; such parameters carry ``_tp_partial_grad`` and
    :func:`reduce_tensor_parallel_grads` sums them over the group before the optimizer step.
  * sequence parallelism: between the linears the activations hold ``tokens / tp`` rows.

Initialisation draws the full tensor with the generator state shared by all ranks and keeps the local slice, so a
tensor-parallel model starts from exactly the weights of the single-device model with the same seed.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn

from ... import ops
from ...enums import Kernel
from ...kernels import is_kernel_allowed
from ...utils import ProcessGroupManager, SafeTensorsWeightsManager, divide_if_divisible
from ...parallel import tensor_parallel as tp
from ..config import CommonConfig, GPTBaseConfig, LadderResidualConfig
from ..layers.activations import get_activation_function, is_glu
from ..layers.attention import Attention
from ..layers.basic import ParameterizedEmbedding, ParameterizedLinear, init_zeros_, loaded_from_checkpoint
from ..layers.mlp import MLP, MoE, ParameterizedExperts, _std
from ..layers.normalization import get_normalization_function
from ..loss import add_aux_loss, clear_aux_loss, get_aux_loss, get_autoregressive_language_modeling_loss, is_aux_loss_zero
from ..modeling import BaseModelMixin, BaseModelOutputWithPast, Block, CausalLMModelMixin, CausalLMOutputWithPast, PreTrainedModelMixin
from ..parameter import mark_parameter_as_mup_learning_rate, mark_parameter_as_no_weight_decay

VOCAB_MULTIPLE = 64


# ----------------------------------------------------------------------------------------------------------------------
# parameter markers and gradient reduction
def mark_tp_sharded(p: nn.Parameter | None, dim: int, parts: int = 1) -> None:
    """``dim``: the sharded dimension; ``parts``: number of equal stacked blocks along it that are each sharded
    (2 for a gated ``c_fc``)."""
    if p is not None:
        p._tp_shard_dim = dim
        p._tp_shard_parts = parts


def mark_tp_partial_grad(p: nn.Parameter | None, when: str) -> None:
    """``when``: "always" or "sequence_parallel"."""
    if p is not None:
        p._tp_partial_grad = when


def reduce_tensor_parallel_grads(model: nn.Module, sequence_parallel: bool) -> None:
    """Sum the gradients of replicated parameters that every rank computed from only its part of the work."""
    if tp.tp_world() == 1:
        return
    grads = []
    for p in model.parameters():
        when = getattr(p, "_tp_partial_grad", None)
        if when == "always" or (when == "sequence_parallel" and sequence_parallel):
            g = getattr(p, "main_grad", None)
            g = p.grad if g is None else g
            if g is not None:
                grads.append(g)
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=tp.tp_group())
    offset = 0
    for g in grads:
        g.copy_(flat[offset : offset + g.numel()].view_as(g))
        offset += g.numel()


def tensor_parallel_vocab_info(vocab_size: int, multiple: int = VOCAB_MULTIPLE) -> tuple[int, int, int]:
    """(first row, one past the last real row, rows per rank) of this rank's vocabulary slice."""
    world, rank = tp.tp_world(), tp.tp_rank()
    divide_if_divisible(multiple, world, "the vocabulary padding multiple must be divisible by the tensor parallel size")
    per_rank = multiple * math.ceil(vocab_size / multiple) // world
    return rank * per_rank, min((rank + 1) * per_rank, vocab_size), per_rank


def _local_slice(full: torch.Tensor, dim: int, parts: int = 1) -> torch.Tensor:
    world, rank = tp.tp_world(), tp.tp_rank()
    if world == 1:
        return full
    if parts == 1:
        return full.chunk(world, dim=dim)[rank]
    blocks = full.chunk(parts, dim=dim)
    return torch.cat([b.chunk(world, dim=dim)[rank] for b in blocks], dim=dim)


@torch.no_grad()
def _init_sliced(param: torch.Tensor, full_shape: tuple[int, ...], std: float, dim: int, parts: int = 1) -> None:
    if loaded_from_checkpoint(param):
        return
    full = torch.empty(full_shape, dtype=torch.float32, device=param.device).normal_(mean=0.0, std=std)
    param.copy_(_local_slice(full, dim, parts))


# ----------------------------------------------------------------------------------------------------------------------
# linears
class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, std: float | None = None,
                 sequence_parallel: bool = False, parts: int = 1) -> None:
        super().__init__()
        self.in_features, self.out_features, self.std, self.parts = in_features, out_features, std, parts
        self.sequence_parallel = sequence_parallel
        self.out_features_per_rank = divide_if_divisible(out_features, tp.tp_world() * parts,
                                                         "output features must be divisible by the tensor parallel size") * parts
        self.weight = nn.Parameter(torch.empty(self.out_features_per_rank, in_features))
        self.bias = nn.Parameter(torch.empty(self.out_features_per_rank)) if bias else None
        mark_tp_sharded(self.weight, 0, parts)
        mark_tp_sharded(self.bias, 0, parts)
        mark_parameter_as_no_weight_decay(self.bias)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        std = self.std if self.std is not None else 1.0 / math.sqrt(self.in_features)
        _init_sliced(self.weight, (self.out_features, self.in_features), std, 0, self.parts)
        init_zeros_(self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel and x.is_cuda and not hasattr(self, "linear_function"):
            from ...parallel import fused_tp

            if fused_tp.fused_ok(x, self.weight, x.shape[0] * tp.tp_world()):
                return fused_tp.ag_linear(x, self.weight, self.bias)  # all-gather inside the GEMM kernel
        x = tp.column_parallel_input(x, self.sequence_parallel)
        return getattr(self, "linear_function", ops.linear)(x, self.weight, self.bias)  # an fp8 recipe replaces the product

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features_per_rank={self.out_features_per_rank}, bias={self.bias is not None}"


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, std: float | None = None,
                 sequence_parallel: bool = False) -> None:
        super().__init__()
        self.in_features, self.out_features, self.std = in_features, out_features, std
        self.sequence_parallel = sequence_parallel
        # True: forward only starts the reduction of the output; whoever consumes it calls tp.finish_reduction (the ladder
        # residual blocks do, one sub-block later, so that the collective runs under that sub-block's compute)
        self.overlap_reduction = False
        self.in_features_per_rank = divide_if_divisible(in_features, tp.tp_world(), "input features must be divisible by the tensor parallel size")
        self.weight = nn.Parameter(torch.empty(out_features, self.in_features_per_rank))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        mark_tp_sharded(self.weight, 1)
        mark_tp_partial_grad(self.bias, "sequence_parallel")
        mark_parameter_as_no_weight_decay(self.bias)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        std = self.std if self.std is not None else 1.0 / math.sqrt(self.in_features)
        _init_sliced(self.weight, (self.out_features, self.in_features), std, 1)
        init_zeros_(self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel and x.is_cuda and not hasattr(self, "linear_function"):
            from ...parallel import fused_tp

            if fused_tp.fused_ok(x, self.weight, x.shape[0]):
                y = fused_tp.linear_rs(x, self.weight)  # reduce-scatter inside the GEMM epilogue
                return y if self.bias is None else y + self.bias
        y = getattr(self, "linear_function", ops.linear)(x, self.weight, None)
        if self.overlap_reduction and self.bias is None:
            return tp.row_parallel_output_async(y, self.sequence_parallel)
        y = tp.row_parallel_output(y, self.sequence_parallel)
        return y if self.bias is None else y + self.bias

    def extra_repr(self) -> str:
        return f"in_features_per_rank={self.in_features_per_rank}, out_features={self.out_features}, bias={self.bias is not None}"


class ReplicatedLinear(ParameterizedLinear):
    """Same weights on every rank; ``partial_grad`` says when its gradient is only this rank's share."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, std: float | None = None,
                 partial_grad: str = "sequence_parallel") -> None:
        super().__init__(in_features, out_features, bias=bias, std=std)
        mark_tp_partial_grad(self.weight, partial_grad)
        mark_tp_partial_grad(self.bias, partial_grad)


def _replicated_norm(name: str | None, size: int, eps: float) -> nn.Module:
    norm = get_normalization_function(name, size, eps=eps)
    for p in norm.parameters():
        mark_tp_partial_grad(p, "sequence_parallel")
    return norm


class Dropout_TP(nn.Dropout):
    """Dropout whose mask differs between ranks where the activations are sharded by tokens (each rank owns other
    tokens) and agrees where they are replicated: sharded regions draw from a generator seeded by the rank."""

    def __init__(self, p: float = 0.5, sequence_parallel: bool = False) -> None:
        super().__init__(p)
        self.sequence_parallel = sequence_parallel
        self._generator: torch.Generator | None = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.training or self.p == 0:
            return x
        if not self.sequence_parallel or tp.tp_world() == 1:
            return super().forward(x)
        if self._generator is None or self._generator.device != x.device:
            self._generator = torch.Generator(device=x.device)
            self._generator.manual_seed(torch.initial_seed() + 7919 * (tp.tp_rank() + 1))
        keep = torch.rand(x.shape, device=x.device, generator=self._generator) >= self.p
        return x * keep.to(x.dtype) / (1.0 - self.p)


def _dropout(p: float, sequence_parallel: bool) -> nn.Module:
    return nn.Identity() if p == 0 else Dropout_TP(p, sequence_parallel)


# ----------------------------------------------------------------------------------------------------------------------
# vocabulary-parallel embedding and LM head
class Embedding_TP(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, std: float | None = None,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.std = num_embeddings, embedding_dim, std
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.vocab_start_index, self.vocab_end_index, per_rank = tensor_parallel_vocab_info(num_embeddings)
        self.weight = nn.Parameter(torch.empty(per_rank, embedding_dim))
        mark_tp_sharded(self.weight, 0)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if loaded_from_checkpoint(self.weight):
            return
        full = torch.empty(self.num_embeddings, self.embedding_dim, dtype=torch.float32, device=self.weight.device)
        full.normal_(mean=0.0, std=self.std if self.std is not None else 1.0)
        self.weight.zero_()  # rows past the real vocabulary (padding) stay zero
        rows = max(self.vocab_end_index - self.vocab_start_index, 0)
        self.weight[:rows].copy_(full[self.vocab_start_index : self.vocab_start_index + rows])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        out = tp.vocab_parallel_embedding(ids, self.weight, self.vocab_start_index)
        return tp.row_parallel_output(out, self.sequence_parallel)


class LMHead_TP(Embedding_TP):
    """Vocabulary-sharded output projection; returns this rank's slice of the logits."""

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.compute_with_weight(hidden_states, self.weight, self.sequence_parallel)

    @staticmethod
    def compute_with_weight(hidden_states: torch.Tensor, weight: torch.Tensor, sequence_parallel: bool) -> torch.Tensor:
        return ops.linear(tp.column_parallel_input(hidden_states, sequence_parallel), weight)


# ----------------------------------------------------------------------------------------------------------------------
# attention
class Attention_TP(Attention):
    """Heads are divided over the ranks; the attention itself is local. Grouped-query attention shards whole key/value
    groups through the fused ``c_attn``; multi-query attention (one key/value head) keeps a column-parallel ``c_attn.q_attn``
    and a replicated ``c_attn.kv_attn`` whose outputs form the local ``[q heads | k | v]`` row."""

    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int, attention_multiplier: float | None,
                 position_embedding_type: str, add_bias: bool, softmax_dropout: float, dropout: float, init_method: str,
                 initializer_range: float, m_width: float | None, num_layers: int, causal: bool, layer_idx: int | None,
                 use_padding_free_transformer: bool, sequence_parallel: bool = False) -> None:
        nn.Module.__init__(self)
        world = tp.tp_world()
        self.causal = causal
        self.global_hidden_size = hidden_size
        self.global_num_heads = num_attention_heads
        self.global_num_key_value_heads = num_key_value_heads
        self.add_bias = add_bias
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.head_dim = divide_if_divisible(hidden_size, num_attention_heads, "hidden_size must be divisible by num_attention_heads")
        self.num_heads = divide_if_divisible(num_attention_heads, world, "num_attention_heads must be divisible by the tensor parallel size")
        self.multi_query = num_key_value_heads == 1 and world > 1
        if self.multi_query:
            self.num_key_value_heads = 1
        else:
            self.num_key_value_heads = divide_if_divisible(num_key_value_heads, world,
                                                           "num_key_value_heads must be 1 or divisible by the tensor parallel size")
        self.group_size = self.num_heads // self.num_key_value_heads
        self.hidden_size = self.num_heads * self.head_dim
        self.position_embedding_type = position_embedding_type
        self.attention_multiplier = attention_multiplier
        self.layer_idx = layer_idx

        std = initializer_range / math.sqrt(m_width) if init_method == "mup" else initializer_range
        if self.multi_query:
            # parameter names as in the reference's tensor-parallel multi-query projection: `c_attn.q_attn`, `c_attn.kv_attn`
            self.c_attn = nn.Module()
            self.c_attn.q_attn = ColumnParallelLinear(hidden_size, hidden_size, bias=add_bias, std=std, sequence_parallel=sequence_parallel)
            self.c_attn.kv_attn = ReplicatedLinear(hidden_size, 2 * self.head_dim, bias=add_bias, std=std, partial_grad="always")
            first = [self.c_attn.q_attn.weight, self.c_attn.kv_attn.weight]
        else:
            self.c_attn = ColumnParallelLinear(hidden_size, hidden_size + 2 * num_key_value_heads * self.head_dim, bias=add_bias,
                                               std=std, sequence_parallel=sequence_parallel)
            first = [self.c_attn.weight]
        std = initializer_range / math.sqrt(2 * num_layers)
        if init_method == "mup":
            std /= math.sqrt(m_width)
        self.c_proj = RowParallelLinear(hidden_size, hidden_size, bias=add_bias, std=std, sequence_parallel=sequence_parallel)
        self.softmax_dropout_p = softmax_dropout
        self.dropout = _dropout(dropout, sequence_parallel)
        for w in first + [self.c_proj.weight]:
            mark_parameter_as_mup_learning_rate(w)

    def forward(self, hidden_states: torch.Tensor, ctx, past_key_values=None) -> torch.Tensor:
        if self.multi_query:
            x = tp.column_parallel_input(hidden_states, self.sequence_parallel)
            qkv = torch.cat([ops.linear(x, self.c_attn.q_attn.weight, self.c_attn.q_attn.bias), self.c_attn.kv_attn(x)], dim=-1)
        else:
            qkv = self.c_attn(hidden_states)
        out = self._forward_packed(qkv, ctx) if ctx.packed else self._forward_padded(qkv, ctx, past_key_values)
        return self.dropout(self.c_proj(out))


# ----------------------------------------------------------------------------------------------------------------------
# MLP and (expert-tensor-parallel) MoE
class MLP_TP(MLP):
    def __init__(self, hidden_size: int, intermediate_size: int, activation_function: str, add_bias: bool, dropout: float,
                 init_method: str, initializer_range: float, m_width: float | None, num_layers: int,
                 sequence_parallel: bool = False) -> None:
        nn.Module.__init__(self)
        self.is_glu = is_glu(activation_function)
        width = 2 if self.is_glu else 1
        self.c_fc = ColumnParallelLinear(hidden_size, width * intermediate_size, bias=add_bias, std=_std(initializer_range, init_method, m_width),
                                         sequence_parallel=sequence_parallel, parts=width)
        self.act = get_activation_function(activation_function)
        self.c_proj = RowParallelLinear(intermediate_size, hidden_size, bias=add_bias,
                                        std=_std(initializer_range, init_method, m_width, num_layers), sequence_parallel=sequence_parallel)
        self.dropout = _dropout(dropout, sequence_parallel)
        mark_parameter_as_mup_learning_rate(self.c_fc.weight)
        mark_parameter_as_mup_learning_rate(self.c_proj.weight)


class _ShardedExperts(ParameterizedExperts):
    """Expert bank of which every rank holds a slice of every expert along ``dim`` (1: outputs, 2: inputs)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool, std: float | None, dim: int, parts: int = 1) -> None:
        self.full_shape = (num_experts, out_features, in_features)
        self.shard_dim, self.parts = dim, parts
        world = tp.tp_world()
        local_in = in_features // world if dim == 2 else in_features
        local_out = out_features // world if dim == 1 else out_features
        divide_if_divisible(out_features if dim == 1 else in_features, world * parts, "expert width must be divisible by the tensor parallel size")
        super().__init__(num_experts, local_in, local_out, add_bias=add_bias, std=std)
        mark_tp_sharded(self.weight, dim, parts)
        if self.bias is not None:
            if dim == 1:
                mark_tp_sharded(self.bias, 1, parts)
            else:
                mark_tp_partial_grad(self.bias, "sequence_parallel")

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if not hasattr(self, "full_shape"):
            return  # called by the parent constructor before the layout is known; called again below
        _init_sliced(self.weight, self.full_shape, self.std if self.std is not None else 0.02, self.shard_dim, self.parts)
        init_zeros_(self.bias)


class MoE_TP(MoE):
    """Every rank computes all experts on all tokens of the group, on its ``intermediate / tp`` slice of each expert;
    the partial outputs are summed (reduce-scatter under sequence parallelism). The router is replicated."""

    def __init__(self, hidden_size: int, intermediate_size: int, shared_intermediate_size: int | None, num_experts: int,
                 num_experts_per_tok: int, activation_function: str, add_bias: bool, dropout: float, init_method: str,
                 initializer_range: float, m_width: float | None, num_layers: int, use_padding_free_transformer: bool,
                 sequence_parallel: bool = False) -> None:
        nn.Module.__init__(self)
        self.expert_parallel = False  # experts are split over the tensor-parallel group here
        self.num_experts, self.top_k = num_experts, num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = divide_if_divisible(intermediate_size, tp.tp_world(), "")
        self.shared_intermediate_size = shared_intermediate_size
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.is_glu = is_glu(activation_function)
        self.activation_function = activation_function
        width = 2 if self.is_glu else 1
        std_in, std_out = _std(initializer_range, init_method, m_width), _std(initializer_range, init_method, m_width, num_layers)

        self.gate = ReplicatedLinear(hidden_size, num_experts, bias=False, std=std_in, partial_grad="sequence_parallel")
        # construction order = order of the single-device module, so that both draw the same random numbers
        self.c_fc = _ShardedExperts(num_experts, hidden_size, width * intermediate_size, add_bias, std_in, dim=1, parts=width)
        if shared_intermediate_size is not None:
            self.c_fc_shared = ColumnParallelLinear(hidden_size, width * shared_intermediate_size, bias=add_bias, std=std_in, parts=width)
        self.act = get_activation_function(activation_function)
        self.c_proj = _ShardedExperts(num_experts, intermediate_size, hidden_size, add_bias, std_out, dim=2)
        if shared_intermediate_size is not None:
            self.c_proj_shared = RowParallelLinear(shared_intermediate_size, hidden_size, bias=add_bias, std=std_out)
        self.dropout = _dropout(dropout, sequence_parallel)
        for module in (self.gate, self.c_fc, self.c_proj):
            mark_parameter_as_mup_learning_rate(module.weight)
        if shared_intermediate_size is not None:
            mark_parameter_as_mup_learning_rate(self.c_fc_shared.weight)
            mark_parameter_as_mup_learning_rate(self.c_proj_shared.weight)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        dim = tp.token_dim(hidden_states)
        logits_local = self.gate(hidden_states)  # on this rank's tokens
        if self.sequence_parallel:
            logits = tp.gather_tokens(logits_local, dim)
            x_full = tp.gather_tokens(hidden_states, dim)
        else:
            logits, x_full = logits_local, tp.copy_to_tp(hidden_states)
        shape = x_full.shape
        x = x_full.reshape(-1, self.hidden_size)
        flat_logits = logits.reshape(-1, self.num_experts)
        if self.top_k == 1:
            top_logits, selected = flat_logits.max(dim=-1, keepdim=True)
        else:
            top_logits, selected = flat_logits.topk(self.top_k, dim=-1)
        weights = torch.softmax(top_logits.float(), dim=-1).type_as(x)
        # Each rank sees the gradient of the routing weights through its slice of the experts only. Under sequence
        # parallelism the backward of the logits gather (a reduce-scatter) already sums those shares; otherwise the
        # sum is made here.
        if not self.sequence_parallel:
            weights = tp.copy_to_tp(weights)
        out = self.experts(x, weights, selected)
        if self.shared_intermediate_size is not None:
            hidden = self.act(ops.linear(x, self.c_fc_shared.weight, self.c_fc_shared.bias))
            out = out + ops.linear(hidden, self.c_proj_shared.weight, None)
        out = tp.row_parallel_output(out.reshape(shape), self.sequence_parallel)
        if self.shared_intermediate_size is not None and self.c_proj_shared.bias is not None:
            out = out + self.c_proj_shared.bias
        out = self.dropout(out)
        if self.training:
            # the auxiliary loss is computed identically on every rank: its gradient must not be summed tp times by
            # the reduce-scatter behind the gathered logits
            aux_logits = _ScaleGradient.apply(logits, 1.0 / tp.tp_world()) if self.sequence_parallel else logits
            self._tokens_per_expert = None
            self._router_statistics(aux_logits, selected)
        return out


class _ScaleGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, factor):
        ctx.factor = factor
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.factor, None


# ----------------------------------------------------------------------------------------------------------------------
# blocks
def _mixer_tp(config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int, sequence_parallel: bool) -> nn.Module:
    block = config.sequence_mixer_blocks[layer_idx]
    if block.sequence_mixer_type != "softmax_attention":
        raise NotImplementedError(f"tensor parallelism covers softmax attention, not {block.sequence_mixer_type}")
    return Attention_TP(hidden_size=config.hidden_size, num_attention_heads=block.num_attention_heads,
                        num_key_value_heads=block.num_key_value_heads, attention_multiplier=block.attention_multiplier,
                        position_embedding_type=config.position_embedding_type, add_bias=block.add_bias,
                        softmax_dropout=block.softmax_dropout, dropout=block.dropout, init_method=config.init_method,
                        initializer_range=config.initializer_range, m_width=config.m_width, num_layers=config.num_layers, causal=True,
                        layer_idx=layer_idx, use_padding_free_transformer=use_padding_free_transformer, sequence_parallel=sequence_parallel)


def _mlp_tp(config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int, sequence_parallel: bool) -> nn.Module:
    block = config.mlp_blocks[layer_idx]
    common = dict(hidden_size=config.hidden_size, intermediate_size=block.intermediate_size, activation_function=block.activation_function,
                  add_bias=block.add_bias, dropout=block.dropout, init_method=config.init_method, initializer_range=config.initializer_range,
                  m_width=config.m_width, num_layers=config.num_layers, sequence_parallel=sequence_parallel)
    if block.mlp_type == "MLP":
        return MLP_TP(**common)
    if block.mlp_type == "MoE":
        return MoE_TP(**common, shared_intermediate_size=block.shared_intermediate_size, num_experts=block.num_experts,
                      num_experts_per_tok=block.num_experts_per_tok, use_padding_free_transformer=use_padding_free_transformer)
    raise ValueError(f"invalid mlp_type ({block.mlp_type}) for layer ({layer_idx})")


class Block_TP(Block):
    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int, sequence_parallel: bool = False) -> None:
        nn.Module.__init__(self)
        self.m_residual = config.m_residual
        self.sequence_mixer_type = config.sequence_mixer_blocks[layer_idx].sequence_mixer_type
        self.layer_idx = layer_idx
        self.ln_1 = _replicated_norm(config.normalization_function, config.hidden_size, config.layer_norm_epsilon)
        self.sequence_mixer = _mixer_tp(config, use_padding_free_transformer, layer_idx, sequence_parallel)
        self.ln_2 = _replicated_norm(config.normalization_function, config.hidden_size, config.layer_norm_epsilon)
        self.mlp_block = _mlp_tp(config, use_padding_free_transformer, layer_idx, sequence_parallel)
        self._fusable = False


class LadderResidualBlock_TP(Block_TP):
    """The block of ``ladder_residual``: the outputs of the previous block join the stream here, one step late, so
    their reductions have the previous sub-block's compute to hide behind."""

    def _overlap(self) -> bool:
        """``Kernel.ladder_residual_overlapped_layer``: the reductions of the two row-parallel projections are started
        and left running; the previous block's attention output is waited for before this block's attention input is
        formed and its MLP output before this block's MLP input, i.e. every reduction has one sub-block of compute to
        hide behind (parity: lm_engine/hf_models/models/ladder_residual_TP/layer.py:140-390 of the reference, which does
        the same with asynchronous functional collectives). Needs projections without bias and without dropout, and
        the plain (not kernel-fused) collectives."""
        plain = lambda module: isinstance(module, nn.Identity) or getattr(module, "p", 0) == 0  # noqa: E731
        ok = (is_kernel_allowed(Kernel.ladder_residual_overlapped_layer) and tp.tp_world() > 1 and self.m_residual is None
              and isinstance(self.mlp_block, MLP_TP) and plain(self.sequence_mixer.dropout) and plain(self.mlp_block.dropout)
              and self.sequence_mixer.c_proj.bias is None and self.mlp_block.c_proj.bias is None
              and not ProcessGroupManager.is_async_tensor_parallel_enabled())
        self.sequence_mixer.c_proj.overlap_reduction = ok
        self.mlp_block.c_proj.overlap_reduction = ok
        return ok

    def forward(self, current_attention_out, current_mlp_out, residual, ctx, past_key_values=None):
        self._overlap()
        if current_attention_out is not None:
            residual = residual + tp.finish_reduction(current_attention_out)
        current_attention_out = self.sequence_mixer(self.ln_1(residual), ctx, past_key_values)
        if self.m_residual is not None:
            current_attention_out = current_attention_out * self.m_residual
        if current_mlp_out is not None:
            residual = residual + tp.finish_reduction(current_mlp_out)
        current_mlp_out = self.mlp_block(self.ln_2(residual))
        if self.m_residual is not None:
            current_mlp_out = current_mlp_out * self.m_residual
        return current_attention_out, current_mlp_out, residual


# ----------------------------------------------------------------------------------------------------------------------
# models
class PreTrainedModelMixin_TP(PreTrainedModelMixin):
    layer_class = Block_TP
    _no_split_modules = ["Block_TP"]

    def __init__(self, config: CommonConfig, *args, **kwargs) -> None:
        self.sequence_parallel = kwargs.pop("sequence_parallel", False)
        self.num_pipeline_stages = kwargs.pop("num_pipeline_stages", 1)
        self.pipeline_stage_id = kwargs.pop("pipeline_stage_id", 0)
        self.is_first_stage = self.pipeline_stage_id == 0
        self.is_last_stage = self.pipeline_stage_id == self.num_pipeline_stages - 1
        self.is_pipeline_parallel_enabled = self.num_pipeline_stages > 1
        super().__init__(config, *args, **kwargs)
        if self.is_pipeline_parallel_enabled and self._tied_word_embeddings:
            raise NotImplementedError("tied word embeddings are not supported with pipeline parallelism")

    def _parallel_kwargs(self) -> dict:
        return dict(use_padding_free_transformer=self.use_padding_free_transformer, sequence_parallel=self.sequence_parallel,
                    num_pipeline_stages=self.num_pipeline_stages, pipeline_stage_id=self.pipeline_stage_id)


class BaseModelMixin_TP(PreTrainedModelMixin_TP, BaseModelMixin):
    def _init_model(self, config: CommonConfig, **kwargs) -> None:
        self.embed_dim = config.hidden_size
        self.m_emb = config.m_emb
        self.initializer_range = config.initializer_range
        self.position_embedding_type = config.position_embedding_type
        self.rope_dim = config.rope_dim

        per_stage = divide_if_divisible(config.num_layers, self.num_pipeline_stages, "layers should be divisible by num_pipeline_stages")
        self.layer_start_id = per_stage * self.pipeline_stage_id
        self.layer_end_id = per_stage * (self.pipeline_stage_id + 1)

        if self.is_first_stage:
            self.wte = Embedding_TP(config.vocab_size, self.embed_dim, std=self.initializer_range,
                                    use_padding_free_transformer=self.use_padding_free_transformer, sequence_parallel=self.sequence_parallel)
            self.embedding_dropout = _dropout(config.embedding_dropout, self.sequence_parallel)
        # keyed by the global layer index so that state-dict names do not depend on the stage
        self.h = nn.ModuleDict({
            str(i): self.layer_class(config, use_padding_free_transformer=self.use_padding_free_transformer, layer_idx=i,
                                     sequence_parallel=self.sequence_parallel)
            for i in range(self.layer_start_id, self.layer_end_id)})
        if self.is_last_stage:
            self.ln_f = _replicated_norm(config.normalization_function, self.embed_dim, config.layer_norm_epsilon)
        self._setup_positional_encoding()
        self.post_init()

    def _setup_positional_encoding(self) -> None:
        if self.position_embedding_type == "learned_absolute":
            if self.is_first_stage:
                # rows divided over the ranks like the token table, which is also the layout of the reference's checkpoints
                self.wpe = Embedding_TP(self.config.max_position_embeddings, self.embed_dim, std=self.initializer_range,
                                        use_padding_free_transformer=self.use_padding_free_transformer,
                                        sequence_parallel=self.sequence_parallel)
        else:
            super()._setup_positional_encoding()

    def _dtype(self) -> torch.dtype:
        return next(self.parameters()).dtype

    def embed(self, input_ids, inputs_embeds, position_ids, token_type_ids) -> torch.Tensor:
        x = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        if self.position_embedding_type == "learned_absolute":
            x = x + self.wpe(position_ids)  # already this rank's tokens under sequence parallelism
        if token_type_ids is not None:
            x = x + self.wte(token_type_ids)
        x = self.embedding_dropout(x)
        if self.m_emb is not None:
            x = x * self.m_emb
        return x

    def run_blocks(self, hidden_states: torch.Tensor, ctx, past_key_values) -> torch.Tensor:
        for block in self.h.values():
            hidden_states = block(hidden_states, ctx, past_key_values)
        return hidden_states

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None, position_ids=None,
                inputs_embeds=None, use_cache=None, cu_seqlens=None, max_seqlen=None) -> BaseModelOutputWithPast:
        """On the first pipeline stage ``input_ids`` are token ids; on later stages they are the hidden states handed
        over by the previous stage (token-sharded under sequence parallelism)."""
        if use_cache is None:
            use_cache = False if self.use_padding_free_transformer else self.config.use_cache
        if self.is_first_stage:
            ctx = self.build_context(input_ids, inputs_embeds, attention_mask, position_ids, past_key_values, cu_seqlens, max_seqlen, self._dtype())
            hidden_states = self.embed(input_ids, inputs_embeds, ctx.position_ids, token_type_ids)
        else:
            hidden_states = input_ids
            ctx = self._context_for_hidden_states(hidden_states, attention_mask, position_ids, past_key_values, cu_seqlens, max_seqlen)
        from ..cache import GenerationCache
        from ..utils import is_generation_cache_enabled

        if is_generation_cache_enabled() and use_cache and past_key_values is None and not self.is_pipeline_parallel_enabled:
            past_key_values = GenerationCache(self.config)
        hidden_states = self.run_blocks(hidden_states, ctx, past_key_values)
        if self.is_last_stage:
            hidden_states = self.ln_f(hidden_states)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=past_key_values)

    def _context_for_hidden_states(self, hidden_states, attention_mask, position_ids, past_key_values, cu_seqlens, max_seqlen):
        """Sequence context of a later pipeline stage: shapes come from the hidden states (times tp under sequence
        parallelism), positions are the plain ranges unless given."""
        if self.use_padding_free_transformer:
            stand_in = torch.empty(0, dtype=torch.long, device=hidden_states.device)  # only its device is looked at
            return self.build_context(stand_in, None, attention_mask, position_ids, past_key_values, cu_seqlens, max_seqlen, hidden_states.dtype)
        batch, length = hidden_states.shape[:2]
        length *= tp.tp_world() if self.sequence_parallel else 1
        stand_in = torch.empty(batch, length, dtype=torch.long, device=hidden_states.device)
        return self.build_context(stand_in, None, attention_mask, position_ids, past_key_values, cu_seqlens, max_seqlen, hidden_states.dtype)


class CausalLMModelMixin_TP(PreTrainedModelMixin_TP, CausalLMModelMixin):
    model_parallel_state_dict_function = None

    def _init_model(self, config: CommonConfig, **kwargs) -> None:
        self.vocab_size = config.vocab_size
        self.transformer = self.base_model_class(config, **self._parallel_kwargs())
        if self.is_last_stage and not self._tied_word_embeddings:
            self.lm_head = LMHead_TP(config.vocab_size, config.hidden_size, std=config.initializer_range,
                                     use_padding_free_transformer=self.use_padding_free_transformer, sequence_parallel=self.sequence_parallel)
        self.post_init()

    def get_lm_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return LMHead_TP.compute_with_weight(hidden_states, self.vocab_projection_weight(), self.sequence_parallel)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None, position_ids=None,
                inputs_embeds=None, labels=None, use_cache=None, return_dict: bool = True, output_parallel_lm_logits: bool = False,
                cu_seqlens=None, max_seqlen=None, reduction: str = "mean", pipeline_parallel_input=None, **unused):
        """Stages other than the last return ``(hidden_states, aux_loss)``; the last returns the usual output with the
        logits either as this rank's vocabulary slice (``output_parallel_lm_logits``) or gathered."""
        assert return_dict
        if not self.is_first_stage:
            assert pipeline_parallel_input is not None, "later pipeline stages take (hidden_states, aux_loss) from the previous one"
            input_ids, aux_in = pipeline_parallel_input
        else:
            aux_in = 0
            input_ids, position_ids, token_type_ids, labels, cu_seqlens, max_seqlen = self.prepare_inputs_for_model(
                input_ids=input_ids, inputs_embeds=inputs_embeds, position_ids=position_ids, token_type_ids=token_type_ids, labels=labels,
                cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, past_key_values=past_key_values, attention_mask=attention_mask, use_cache=use_cache)

        clear_aux_loss()
        if not is_aux_loss_zero(aux_in):
            add_aux_loss(aux_in)
        outputs = self.transformer(input_ids, past_key_values=past_key_values, attention_mask=attention_mask, token_type_ids=token_type_ids,
                                   position_ids=position_ids, inputs_embeds=inputs_embeds, use_cache=use_cache, cu_seqlens=cu_seqlens,
                                   max_seqlen=max_seqlen)
        hidden_states = outputs.last_hidden_state
        aux_loss = get_aux_loss()
        if not self.is_last_stage:
            if is_aux_loss_zero(aux_loss):
                aux_loss = torch.zeros((), device=hidden_states.device, dtype=torch.float32)
            return hidden_states, aux_loss

        lm_logits = self.get_lm_logits(hidden_states)
        if self.m_width is not None:
            lm_logits = lm_logits / self.m_width
        start, end, per_rank = tensor_parallel_vocab_info(self.vocab_size)
        if end - start < per_rank:  # columns of the vocabulary padding must not take part in the softmax
            padding = torch.arange(per_rank, device=lm_logits.device) >= max(end - start, 0)
            lm_logits = lm_logits.masked_fill(padding, float("-inf"))
        loss = None
        if labels is not None:
            loss = get_autoregressive_language_modeling_loss(
                lm_logits=lm_logits, labels=labels, cu_seqlens=cu_seqlens, use_padding_free_transformer=self.use_padding_free_transformer,
                reduction=reduction, shift_logits_and_labels=True, tensor_parallel_enabled=tp.tp_world() > 1)
            if not is_aux_loss_zero(aux_loss):
                loss = loss + self.router_aux_loss_coef * aux_loss
        if not output_parallel_lm_logits:
            lm_logits = tp.gather_features(lm_logits)[..., : self.vocab_size]
        return CausalLMOutputWithPast(loss=loss, aux_loss=aux_loss, logits=lm_logits, past_key_values=outputs.past_key_values,
                                      last_hidden_state=hidden_states)

    # ------------------------------------------------------------------ weights
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, dtype: torch.dtype = torch.float32, **kwargs):
        """Builds the local part of the model and fills it from the safetensors files of an unsharded checkpoint; every
        rank reads only the slices it owns."""
        from ...utils import download_repo

        config, _, weights_path = download_repo(pretrained_model_name_or_path)
        if not isinstance(config, cls.config_class):
            config = cls.config_class.from_pretrained(pretrained_model_name_or_path)
        model = cls._from_config(config, **kwargs)
        model.load_from_safetensors_weights_manager(SafeTensorsWeightsManager(weights_path))
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        return model.to(device=device, dtype=dtype)

    @classmethod
    def _from_config(cls, config, **kwargs):
        kwargs.pop("torch_dtype", None)
        kwargs.pop("attn_implementation", None)
        return cls(config, **kwargs)

    def load_from_safetensors_weights_manager(self, manager: SafeTensorsWeightsManager) -> None:
        state = type(self).model_parallel_state_dict_function(
            config=self.config, safetensors_weights_manager=manager, num_pipeline_stages=self.num_pipeline_stages,
            pipeline_stage_id=self.pipeline_stage_id)
        self.load_state_dict(state)


# ----------------------------------------------------------------------------------------------------------------------
# concrete families
def _gpt_base_parallel_state_dict(**kwargs):
    from ..tp_weights import get_gpt_base_model_parallel_state_dict

    return get_gpt_base_model_parallel_state_dict(**kwargs)


class GPTBasePreTrainedModel_TP(PreTrainedModelMixin_TP):
    config_class = GPTBaseConfig


class GPTBaseModel_TP(GPTBasePreTrainedModel_TP, BaseModelMixin_TP):
    pass


class GPTBaseForCausalLM_TP(GPTBasePreTrainedModel_TP, CausalLMModelMixin_TP):
    base_model_class = GPTBaseModel_TP
    model_parallel_state_dict_function = staticmethod(_gpt_base_parallel_state_dict)


class LadderResidualPreTrainedModel_TP(PreTrainedModelMixin_TP):
    config_class = LadderResidualConfig
    layer_class = LadderResidualBlock_TP
    _no_split_modules = ["LadderResidualBlock_TP"]


class LadderResidualModel_TP(LadderResidualPreTrainedModel_TP, BaseModelMixin_TP):
    def run_blocks(self, hidden_states: torch.Tensor, ctx, past_key_values) -> torch.Tensor:
        attention_out = mlp_out = None
        residual = hidden_states
        for block in self.h.values():
            attention_out, mlp_out, residual = block(attention_out, mlp_out, residual, ctx, past_key_values)
        return residual + tp.finish_reduction(attention_out) + tp.finish_reduction(mlp_out)


class LadderResidualForCausalLM_TP(LadderResidualPreTrainedModel_TP, CausalLMModelMixin_TP):
    base_model_class = LadderResidualModel_TP
    model_parallel_state_dict_function = staticmethod(_gpt_base_parallel_state_dict)

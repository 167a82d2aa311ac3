"""Per-layer factories (parity: lm_engine/hf_models/modeling_utils/sequence_mixer_blocks/__init__.py:22-134 and
mlp_blocks/__init__.py:10-39)."""

from __future__ import annotations

import torch.nn as nn

from ..config import CommonConfig
from .attention import Attention
from .mlp import MLP, MoE


def get_mlp_block(config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int) -> nn.Module:
    block = config.mlp_blocks[layer_idx]
    common = dict(
        hidden_size=config.hidden_size, intermediate_size=block.intermediate_size,
        activation_function=block.activation_function, add_bias=block.add_bias, dropout=block.dropout,
        init_method=config.init_method, initializer_range=config.initializer_range, m_width=config.m_width,
        num_layers=config.num_layers,
    )
    if block.mlp_type == "MLP":
        return MLP(**common)
    if block.mlp_type == "MoE":
        return MoE(**common, shared_intermediate_size=block.shared_intermediate_size, num_experts=block.num_experts,
                   num_experts_per_tok=block.num_experts_per_tok, use_padding_free_transformer=use_padding_free_transformer)
    raise ValueError(f"invalid mlp_type ({block.mlp_type}) for layer ({layer_idx})")


def get_sequence_mixer(config: CommonConfig, causal: bool, use_padding_free_transformer: bool, layer_idx: int) -> nn.Module:
    block = config.sequence_mixer_blocks[layer_idx]
    kind = block.sequence_mixer_type
    shared = dict(init_method=config.init_method, initializer_range=config.initializer_range, m_width=config.m_width,
                  num_layers=config.num_layers, layer_idx=layer_idx, use_padding_free_transformer=use_padding_free_transformer)

    if kind == "softmax_attention":
        return Attention(hidden_size=config.hidden_size, num_attention_heads=block.num_attention_heads,
                         num_key_value_heads=block.num_key_value_heads, attention_multiplier=block.attention_multiplier,
                         position_embedding_type=config.position_embedding_type, add_bias=block.add_bias,
                         softmax_dropout=block.softmax_dropout, dropout=block.dropout, causal=causal, **shared)
    if kind == "stickbreaking_attention":
        from .stickbreaking import StickBreakingAttention

        return StickBreakingAttention(hidden_size=config.hidden_size, num_attention_heads=block.num_attention_heads,
                                      num_key_value_heads=block.num_key_value_heads,
                                      attention_multiplier=block.attention_multiplier, add_bias=block.add_bias,
                                      dropout=block.dropout, causal=causal, **shared)
    if kind == "multihead_latent_attention":
        from .latent_attention import MultiHeadLatentAttention

        return MultiHeadLatentAttention(hidden_size=config.hidden_size, query_compression_size=block.query_compression_size,
                                        key_value_compression_size=block.key_value_compression_size,
                                        num_attention_heads=block.num_attention_heads, head_dim=block.head_dim,
                                        attention_multiplier=block.attention_multiplier,
                                        position_embedding_type=config.position_embedding_type, add_bias=block.add_bias,
                                        softmax_dropout=block.softmax_dropout, dropout=block.dropout, causal=causal,
                                        normalization_function=block.normalization_function,
                                        layer_norm_epsilon=config.layer_norm_epsilon, **shared)
    if kind == "mamba2":
        from .mamba2 import Mamba2

        return Mamba2(hidden_size=config.hidden_size, ssm_state_size=block.state_size,
                      ssm_intermediate_size=block.intermediate_size, ssm_num_heads=block.num_heads,
                      conv_kernel_size=block.conv_kernel_size, time_step_limit=block.time_step_limit,
                      add_bias=block.add_bias, use_conv_bias=block.use_conv_bias,
                      ssm_activation_function=block.activation_function, num_groups=block.num_groups,
                      chunk_size=block.chunk_size, layer_norm_epsilon=config.layer_norm_epsilon,
                      initializer_range=config.initializer_range, init_method=config.init_method, m_width=config.m_width,
                      num_layers=config.num_layers, layer_idx=layer_idx)
    if kind in ("gru", "rnn"):
        from .recurrent import GRU, RNN

        cls = GRU if kind == "gru" else RNN
        return cls(input_size=config.hidden_size, state_size=block.state_size, output_size=config.hidden_size,
                   num_heads=block.num_heads, add_bias=block.add_bias, gradient_clipping=block.gradient_clipping,
                   normalization_function=block.normalization_function, layer_norm_epsilon=config.layer_norm_epsilon, **shared)
    if kind == "causal_convolution":
        from .causal_convolution import CausalConvolution

        return CausalConvolution(hidden_size=config.hidden_size, in_channels=block.in_channels,
                                 out_channels=block.out_channels, kernel_size=block.kernel_size,
                                 num_groups=block.num_groups, activation_function=block.activation_function,
                                 add_bias=block.add_bias, **shared)
    raise ValueError(f"unexpected sequence_mixer_type ({kind})")

"""Decoder-only model family: pre-norm blocks of (sequence mixer, MLP/MoE) over a token embedding.

Parity: lm_engine/hf_models/mixins/dense/{base.py, layer.py, main.py} and mixins/modeling_outputs.py. Module and
parameter names (``transformer.wte``, ``transformer.h.{i}.ln_1``, ``.sequence_mixer.c_attn``, ``.mlp_block.c_fc`` ...,
``transformer.ln_f``, ``lm_head``) define the checkpoint format and are kept.

Inputs are either padded ``[batch, seq]`` tensors with an optional ``attention_mask``, or padding-free: nested
lists of token ids, or a flat ``[T]`` tensor with ``cu_seqlens``, ``max_seqlen`` and ``position_ids``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from transformers import GenerationMixin, PreTrainedModel
from transformers.modeling_outputs import ModelOutput

from .. import ops
from ..enums import Kernel
from ..kernels import is_kernel_allowed
from .cache import GenerationCache
from .config import CommonConfig
from .context import SequenceContext
from .layers.basic import ParameterizedEmbedding, ParameterizedLinear
from .layers.mixers import get_mlp_block, get_sequence_mixer
from .layers.normalization import get_normalization_function
from .layers.rope import RoPE, YaRNScaledRoPE
from .loss import clear_aux_loss, get_aux_loss, get_autoregressive_language_modeling_loss, is_aux_loss_zero
from .utils import convert_padding_free_lists_to_tensors, is_generation_cache_enabled


@dataclass
class BaseModelOutputWithPast(ModelOutput):
    last_hidden_state: torch.Tensor | None = None
    past_key_values: GenerationCache | None = None


@dataclass
class CausalLMOutputWithPast(ModelOutput):
    loss: torch.Tensor | None = None
    aux_loss: torch.Tensor | float | None = None
    logits: torch.Tensor | None = None
    past_key_values: GenerationCache | None = None
    last_hidden_state: torch.Tensor | None = None


@dataclass
class PipelineParallelInput(ModelOutput):
    hidden_states: torch.Tensor | None = None
    aux_loss: torch.Tensor | float = 0


@dataclass
class PipelineParallelOutput(ModelOutput):
    hidden_states: torch.Tensor | None = None
    aux_loss: torch.Tensor | float = 0


class Block(nn.Module):
    """``x + m_residual * mixer(ln_1(x))`` followed by ``x + m_residual * mlp(ln_2(x))``."""

    def __init__(self, config: CommonConfig, use_padding_free_transformer: bool, layer_idx: int | None = None) -> None:
        super().__init__()
        self.m_residual = config.m_residual
        self.sequence_mixer_type = config.sequence_mixer_blocks[layer_idx].sequence_mixer_type
        self.layer_idx = layer_idx
        self.ln_1 = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.sequence_mixer = get_sequence_mixer(config, True, use_padding_free_transformer, layer_idx)
        self.ln_2 = get_normalization_function(config.normalization_function, config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp_block = get_mlp_block(config, use_padding_free_transformer=use_padding_free_transformer, layer_idx=layer_idx)
        self._fusable = self._statically_fusable(config, layer_idx)

    def _statically_fusable(self, config: CommonConfig, layer_idx: int) -> bool:
        """The whole-block kernel schedule covers: RMSNorm, bias-free softmax attention with head width 64/128 and
        rope/nope positions, bias-free SwiGLU MLP, no dropout, no residual multiplier."""
        mixer = config.sequence_mixer_blocks[layer_idx]
        mlp = config.mlp_blocks[layer_idx]
        if config.normalization_function != "rmsnorm" or config.m_residual is not None:
            return False
        if mixer.sequence_mixer_type != "softmax_attention" or mlp.mlp_type != "MLP":
            return False
        if mixer.add_bias or mixer.dropout != 0 or mixer.softmax_dropout != 0:
            return False
        if mlp.add_bias or mlp.dropout != 0 or mlp.activation_function != "swiglu":
            return False
        head_dim = config.hidden_size // mixer.num_attention_heads
        if head_dim not in (64, 128) or config.position_embedding_type not in ("rope", "nope"):
            return False
        if config.position_embedding_type == "rope" and (config.rope_dim % 16 != 0 or config.rope_dim > head_dim):
            return False
        return config.hidden_size % 8 == 0 and mlp.intermediate_size % 8 == 0

    def _forward_fused(self, x: torch.Tensor, ctx: SequenceContext) -> torch.Tensor:
        from ..ops.fused_block import fused_dense_block

        att = self.sequence_mixer
        cos = sin = None
        rope_dim = 0
        if att.position_embedding_type == "rope":
            cos, sin = ctx.rope_half_tables
            rope_dim = cos.shape[-1] * 2
        pos = None if ctx.position_ids is None else ctx.position_ids_int32()
        return fused_dense_block(
            x, self.ln_1.weight, att.c_attn.weight, att.c_proj.weight, self.ln_2.weight, self.mlp_block.c_fc.weight,
            self.mlp_block.c_proj.weight, cos, sin, pos, ctx.cu_seqlens_int32(), ctx.max_seqlen,
            att.num_key_value_heads, att.group_size, att.head_dim, rope_dim, att.softmax_scale, self.ln_1.eps)

    def forward(self, hidden_states: torch.Tensor, ctx: SequenceContext, past_key_values: GenerationCache | None = None) -> torch.Tensor:
        if (self._fusable and ctx.packed and past_key_values is None and hidden_states.is_cuda
                and hidden_states.dtype == torch.bfloat16 and hidden_states.dim() == 2
                and is_kernel_allowed(Kernel.fused_block) and ops.native_available()):
            return self._forward_fused(hidden_states.contiguous(), ctx)
        residual = hidden_states
        hidden_states = self.ln_1(hidden_states)
        hidden_states = self.sequence_mixer(hidden_states, ctx, past_key_values)
        if self.m_residual is not None:
            hidden_states = hidden_states * self.m_residual
        hidden_states = hidden_states + residual

        residual = hidden_states
        hidden_states = self.ln_2(hidden_states)
        hidden_states = self.mlp_block(hidden_states)
        if self.m_residual is not None:
            hidden_states = hidden_states * self.m_residual
        return hidden_states + residual


class PreTrainedModelMixin(PreTrainedModel):
    config_class = None
    layer_class = Block
    base_model_prefix = "transformer"
    causal = True
    _no_split_modules = ["Block"]
    _skip_keys_device_placement = "past_key_values"
    supports_gradient_checkpointing = True
    _supports_sdpa = True
    _supports_flash_attn = True

    def __init__(self, config: CommonConfig, *args, **kwargs) -> None:
        self.use_padding_free_transformer = kwargs.pop("use_padding_free_transformer", False)
        super().__init__(config, *args)
        assert self.config_class is not None
        self._tied_word_embeddings = config.tie_word_embeddings
        self._has_linear_mixer = any(b.sequence_mixer_type in ("mamba2", "rnn", "gru") for b in config.sequence_mixer_blocks)

    def _init_weights(self, module: nn.Module) -> None:
        if hasattr(module, "reset_parameters"):
            module.reset_parameters()

    def prepare_inputs_for_model(self, input_ids, inputs_embeds, position_ids, token_type_ids, labels, cu_seqlens,
                                 max_seqlen, past_key_values, attention_mask, use_cache):
        if self.use_padding_free_transformer:
            if isinstance(input_ids, list) or isinstance(inputs_embeds, list):
                for name, value in (("cu_seqlens", cu_seqlens), ("max_seqlen", max_seqlen), ("attention_mask", attention_mask)):
                    if value is not None:
                        raise ValueError(f"{name} is derived internally when the inputs are nested lists")
                device = next(self.parameters()).device
                input_ids, position_ids, token_type_ids, labels, cu_seqlens, max_seqlen = convert_padding_free_lists_to_tensors(
                    input_ids=input_ids, inputs_embeds=inputs_embeds, position_ids=position_ids,
                    token_type_ids=token_type_ids, labels=labels, device=device)
            else:
                if cu_seqlens is None or max_seqlen is None or position_ids is None:
                    raise ValueError("packed tensor inputs need cu_seqlens, max_seqlen and position_ids")
                if attention_mask is not None:
                    raise ValueError("attention_mask can't be combined with cu_seqlens")
            if use_cache or past_key_values is not None:
                raise NotImplementedError("KV caching is not supported with the padding-free transformer")
        return input_ids, position_ids, token_type_ids, labels, cu_seqlens, max_seqlen


class BaseModelMixin(PreTrainedModelMixin):
    def __init__(self, config: CommonConfig, **kwargs) -> None:
        super().__init__(config, **kwargs)
        self._init_model(config, **kwargs)

    def _init_model(self, config: CommonConfig, **kwargs) -> None:
        self.embed_dim = config.hidden_size
        self.m_emb = config.m_emb
        self.initializer_range = config.initializer_range
        self.position_embedding_type = config.position_embedding_type
        self.rope_dim = config.rope_dim

        self.wte = ParameterizedEmbedding(config.vocab_size, self.embed_dim, std=self.initializer_range)
        self.embedding_dropout = nn.Identity() if config.embedding_dropout == 0 else nn.Dropout(config.embedding_dropout)
        self.h = nn.ModuleList(
            [self.layer_class(config, use_padding_free_transformer=self.use_padding_free_transformer, layer_idx=i)
             for i in range(config.num_layers)]
        )
        self.ln_f = get_normalization_function(config.normalization_function, self.embed_dim, eps=config.layer_norm_epsilon)
        self._setup_positional_encoding()
        self.post_init()

    def _setup_positional_encoding(self) -> None:
        cfg = self.config
        if self.position_embedding_type == "learned_absolute":
            self.wpe = ParameterizedEmbedding(cfg.max_position_embeddings, self.embed_dim, std=self.initializer_range)
        elif self.position_embedding_type == "rope":
            yarn = cfg.yarn_scaling()
            if yarn is None:
                self.rope = RoPE(self.rope_dim, max_position_embeddings=cfg.max_position_embeddings, base=cfg.rope_theta)
            else:
                self.rope = YaRNScaledRoPE(
                    self.rope_dim, max_position_embeddings=cfg.max_position_embeddings, base=cfg.rope_theta,
                    scale=yarn["factor"], original_max_position_embeddings=yarn["original_max_position_embeddings"])

    def get_input_embeddings(self):
        return self.wte

    def set_input_embeddings(self, value) -> None:
        self.wte = value

    # ------------------------------------------------------------------ input preparation
    def build_context(self, input_ids, inputs_embeds, attention_mask, position_ids, past_key_values, cu_seqlens,
                      max_seqlen, dtype) -> SequenceContext:
        ref = input_ids if input_ids is not None else inputs_embeds
        if ref is None:
            raise ValueError("either input_ids or inputs_embeds must be given")
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("input_ids and inputs_embeds are mutually exclusive")
        device = ref.device

        if self.use_padding_free_transformer:
            if isinstance(max_seqlen, torch.Tensor):
                max_seqlen = int(max_seqlen.item())
            ctx = SequenceContext(packed=True, batch_size=cu_seqlens.shape[0] - 1, query_length=max_seqlen,
                                  key_length=max_seqlen, position_ids=position_ids, cu_seqlens=cu_seqlens,
                                  max_seqlen=max_seqlen)
            table_len = max(max_seqlen, self.config.max_position_embeddings)
        else:
            batch, query_length = (input_ids.shape if input_ids is not None else inputs_embeds.shape[:2])
            past = 0 if past_key_values is None else past_key_values.get_seq_length()
            key_length = past + query_length
            if position_ids is None:
                if attention_mask is not None and attention_mask.dim() == 2:
                    position_ids = attention_mask.long().cumsum(-1) - 1
                    position_ids.masked_fill_(attention_mask == 0, 0)
                    position_ids = position_ids[:, past:key_length]
                else:
                    position_ids = torch.arange(past, key_length, dtype=torch.long, device=device).unsqueeze(0)
            ctx = SequenceContext(packed=False, batch_size=batch, query_length=query_length, key_length=key_length,
                                  position_ids=position_ids, attention_mask=attention_mask)
            table_len = key_length

        if self.position_embedding_type == "rope":
            ctx.rope_half_tables = self.rope.half_tables(table_len, device)
            if not ctx.packed:
                cos, sin = self.rope(table_len, dtype=dtype, device=device)
                ctx.rope_cos_sin = (cos[ctx.position_ids].unsqueeze(1), sin[ctx.position_ids].unsqueeze(1))
        return ctx

    def embed(self, input_ids, inputs_embeds, position_ids, token_type_ids) -> torch.Tensor:
        x = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        if self.position_embedding_type == "learned_absolute":
            x = x + self.wpe(position_ids)
        if token_type_ids is not None:
            x = x + self.wte(token_type_ids)
        x = self.embedding_dropout(x)
        if self.m_emb is not None:
            x = x * self.m_emb
        return x

    def _linear_mixer_mask(self, attention_mask, past_key_values):
        if attention_mask is None or (past_key_values is not None and past_key_values.get_seq_length() > 0):
            return None
        return None if bool(torch.all(attention_mask == 1)) else attention_mask

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None,
                position_ids=None, inputs_embeds=None, use_cache=None, cu_seqlens=None, max_seqlen=None) -> BaseModelOutputWithPast:
        if use_cache is None:
            use_cache = False if self.use_padding_free_transformer else self.config.use_cache
        dtype = self.wte.weight.dtype
        ctx = self.build_context(input_ids, inputs_embeds, attention_mask, position_ids, past_key_values, cu_seqlens,
                                 max_seqlen, dtype)
        hidden_states = self.embed(input_ids, inputs_embeds, ctx.position_ids, token_type_ids)

        if is_generation_cache_enabled() and use_cache and past_key_values is None:
            past_key_values = GenerationCache(self.config)

        for block in self.h:
            hidden_states = block(hidden_states, ctx, past_key_values)
        hidden_states = self.ln_f(hidden_states)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=past_key_values)


class CausalLMModelMixin(PreTrainedModelMixin, GenerationMixin):
    base_model_class = None
    _tied_weights_keys = {}

    def __init__(self, config: CommonConfig, **kwargs) -> None:
        super().__init__(config, **kwargs)
        self.router_aux_loss_coef = getattr(config, "router_aux_loss_coef", 0)
        self.m_width = config.m_width
        self._init_model(config, **kwargs)

    def _init_model(self, config: CommonConfig, **kwargs) -> None:
        self.transformer = self.base_model_class(config, use_padding_free_transformer=self.use_padding_free_transformer)
        if not self._tied_word_embeddings:
            self.lm_head = ParameterizedLinear(config.hidden_size, config.vocab_size, bias=False, std=config.initializer_range)
        self.post_init()

    def get_input_embeddings(self):
        return self.transformer.wte

    def set_input_embeddings(self, value) -> None:
        self.transformer.wte = value

    def get_output_embeddings(self):
        return self.transformer.wte if self._tied_word_embeddings else self.lm_head

    def set_output_embeddings(self, new_embeddings) -> None:
        if not self._tied_word_embeddings:
            self.lm_head = new_embeddings

    def tie_weights(self, *args, **kwargs) -> None:  # weights are tied by construction (the embedding is reused)
        return None

    def vocab_projection_weight(self) -> torch.Tensor:
        return self.transformer.wte.weight if self._tied_word_embeddings else self.lm_head.weight

    def get_lm_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden_states, self.vocab_projection_weight())

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None,
                position_ids=None, inputs_embeds=None, labels=None, use_cache=None, return_dict: bool = True,
                cu_seqlens=None, max_seqlen=None, reduction: str = "mean", **unused) -> CausalLMOutputWithPast:
        assert return_dict
        input_ids, position_ids, token_type_ids, labels, cu_seqlens, max_seqlen = self.prepare_inputs_for_model(
            input_ids=input_ids, inputs_embeds=inputs_embeds, position_ids=position_ids, token_type_ids=token_type_ids,
            labels=labels, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, past_key_values=past_key_values,
            attention_mask=attention_mask, use_cache=use_cache)

        clear_aux_loss()
        outputs = self.transformer(input_ids, past_key_values=past_key_values, attention_mask=attention_mask,
                                   token_type_ids=token_type_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                                   use_cache=use_cache, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
        hidden_states = outputs.last_hidden_state
        past_key_values = outputs.past_key_values

        fused = is_kernel_allowed(Kernel.fused_linear_cross_entropy_cute)
        logit_scale = 1.0 if self.m_width is None else 1.0 / self.m_width
        lm_logits = None
        loss = None
        if labels is None:
            if fused:
                # callers that enable the fused kernel compute the loss themselves from the hidden states
                if self.m_width is not None:
                    hidden_states = hidden_states / self.m_width
            else:
                lm_logits = self.get_lm_logits(hidden_states)
                if self.m_width is not None:
                    lm_logits = lm_logits / self.m_width
        elif fused:
            loss = get_autoregressive_language_modeling_loss(
                lm_logits=None, labels=labels, hidden_states=hidden_states, vocab_weight=self.vocab_projection_weight(),
                cu_seqlens=cu_seqlens, use_padding_free_transformer=self.use_padding_free_transformer,
                reduction=reduction, shift_logits_and_labels=True, logit_scale=logit_scale)
        else:
            lm_logits = self.get_lm_logits(hidden_states)
            if self.m_width is not None:
                lm_logits = lm_logits / self.m_width
            loss = get_autoregressive_language_modeling_loss(
                lm_logits=lm_logits, labels=labels, cu_seqlens=cu_seqlens,
                use_padding_free_transformer=self.use_padding_free_transformer, reduction=reduction,
                shift_logits_and_labels=True)

        aux_loss = get_aux_loss()
        if loss is not None and not is_aux_loss_zero(aux_loss):
            loss = loss + self.router_aux_loss_coef * aux_loss
        return CausalLMOutputWithPast(loss=loss, aux_loss=aux_loss, logits=lm_logits, past_key_values=past_key_values,
                                      last_hidden_state=hidden_states)

    # ------------------------------------------------------------------ generation plumbing
    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, inputs_embeds=None,
                                      position_ids=None, **kwargs):
        if past_key_values is not None and past_key_values.get_seq_length() > 0:
            input_ids = input_ids[:, past_key_values.get_seq_length():]
            position_ids = None
        model_inputs = {"input_ids": input_ids, "past_key_values": past_key_values, "attention_mask": attention_mask,
                        "use_cache": kwargs.get("use_cache", True), "position_ids": position_ids}
        if inputs_embeds is not None and (past_key_values is None or past_key_values.get_seq_length() == 0):
            model_inputs["inputs_embeds"] = inputs_embeds
            model_inputs["input_ids"] = None
        return model_inputs

    def _reorder_cache(self, past_key_values, beam_idx):
        past_key_values.reorder_cache(beam_idx)
        return past_key_values

    @torch.no_grad()
    def generate(self, inputs=None, attention_mask=None, max_new_tokens: int = 20, do_sample: bool = False,
                 temperature: float | None = None, top_k: int | None = None, top_p: float | None = None,
                 eos_token_id: int | None = None, pad_token_id: int | None = None, return_dict_in_generate: bool = False,
                 output_scores: bool = False, input_ids=None, **kwargs):
        """Greedy / sampling decoding with the generation cache (padded, left-padded prompts).

        Returns the full sequences ``[batch, prompt + new]``; with ``return_dict_in_generate`` a small namespace
        with ``sequences`` and (optionally) per-step ``scores``.
        """
        from .generation import decode

        ids = inputs if inputs is not None else input_ids
        return decode(self, ids, attention_mask, max_new_tokens, do_sample, temperature, top_k, top_p,
                      self.config.eos_token_id if eos_token_id is None else eos_token_id,
                      self.config.pad_token_id if pad_token_id is None else pad_token_id,
                      return_dict_in_generate, output_scores)

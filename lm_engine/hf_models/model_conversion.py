"""Import from / export to Hugging Face checkpoints: pure tensor re-layouts over safetensors files.

Parity: lm_engine/hf_models/model_conversion/{__init__,llama,granite,granitemoe,granitemoeshared,
granitemoesharedhybrid,bigcode}.py. Supported HF ``model_type``s: ``llama``, ``granite``, ``granitemoe``,
``granitemoeshared``, ``granitemoehybrid``, ``gpt_bigcode``.

Layout contracts:
  * attention: HF keeps q/k/v separately; here ``c_attn`` stacks them per key/value group ``[q heads of group | k | v]``
    (``[q | k | v]`` per head for MHA, ``[Q; k; v]`` for MQA which is also gpt_bigcode's native layout);
  * gated MLP: here ``c_fc = [up; gate]`` and the activation is ``up * act(gate)``; Llama/Granite store ``gate_proj``
    and ``up_proj`` separately, Granite-MoE stores ``input_linear = [gate; up]`` (halves swapped);
  * Granite multipliers: ``embedding_multiplier <-> m_emb``, ``residual_multiplier <-> m_residual``,
    ``logits_scaling <-> m_width``, ``attention_multiplier`` per attention block;
  * ``granitemoehybrid``: ``mamba`` layers <-> ``mamba2`` blocks, position embedding ``nope``.
"""

from __future__ import annotations

import os

import torch
from transformers import AutoConfig, AutoTokenizer

from ..utils import SafeTensorsWeightsManager, download_repo
from .config import GPTBaseConfig
from .layers.attention import interleave_query_key_value_tensor_for_attention, split_query_key_value_tensor_for_attention

_LLAMA_LIKE = ("llama", "granite", "granitemoe", "granitemoeshared", "granitemoehybrid")


# ----------------------------------------------------------------------------------------------------------------------
# config translation
def _layer_kinds(hf) -> list[str]:
    if hf.model_type == "granitemoehybrid":
        return ["mamba2" if t == "mamba" else "softmax_attention" for t in hf.layer_types]
    return ["softmax_attention"] * hf.num_hidden_layers


def _import_config(hf) -> GPTBaseConfig:
    if hf.model_type == "gpt_bigcode":
        n = hf.n_layer
        heads = hf.n_head
        attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=heads,
                    num_key_value_heads=1 if hf.multi_query else heads, add_bias=True,
                    attention_multiplier=None if hf.scale_attn_weights else 1.0, softmax_dropout=hf.attn_pdrop, dropout=hf.resid_pdrop)
        mlp = dict(mlp_type="MLP", intermediate_size=hf.n_inner or 4 * hf.n_embd, activation_function=hf.activation_function,
                   add_bias=True, dropout=hf.resid_pdrop)
        return GPTBaseConfig(
            vocab_size=hf.vocab_size, max_position_embeddings=hf.n_positions, hidden_size=hf.n_embd, num_layers=n,
            embedding_dropout=hf.embd_pdrop, normalization_function="layernorm", layer_norm_epsilon=hf.layer_norm_epsilon,
            initializer_range=hf.initializer_range, use_cache=hf.use_cache, position_embedding_type="learned_absolute",
            tie_word_embeddings=True, bos_token_id=hf.bos_token_id, eos_token_id=hf.eos_token_id, pad_token_id=hf.pad_token_id,
            sequence_mixer_blocks=[dict(attn) for _ in range(n)], mlp_blocks=[dict(mlp) for _ in range(n)])

    if hf.model_type not in _LLAMA_LIKE:
        raise NotImplementedError(f"the current model_type ({hf.model_type}) is not yet supported")
    n = hf.num_hidden_layers
    kinds = _layer_kinds(hf)
    is_moe = hf.model_type in ("granitemoe", "granitemoeshared", "granitemoehybrid")
    mixers, mlps = [], []
    for kind in kinds:
        if kind == "mamba2":
            mixers.append(dict(sequence_mixer_type="mamba2", state_size=hf.mamba_d_state, num_heads=hf.mamba_n_heads,
                               intermediate_size=hf.mamba_expand * hf.hidden_size, conv_kernel_size=hf.mamba_d_conv,
                               add_bias=hf.mamba_proj_bias, use_conv_bias=hf.mamba_conv_bias, num_groups=hf.mamba_n_groups,
                               chunk_size=hf.mamba_chunk_size, activation_function=hf.hidden_act))
        else:
            mixers.append(dict(sequence_mixer_type="softmax_attention", num_attention_heads=hf.num_attention_heads,
                               num_key_value_heads=hf.num_key_value_heads, add_bias=getattr(hf, "attention_bias", False),
                               attention_multiplier=getattr(hf, "attention_multiplier", None) if hf.model_type != "llama" else None,
                               softmax_dropout=getattr(hf, "attention_dropout", 0)))
        if is_moe and getattr(hf, "num_local_experts", 0) > 0:
            shared = getattr(hf, "shared_intermediate_size", None)
            mlps.append(dict(mlp_type="MoE", intermediate_size=hf.intermediate_size, num_experts=hf.num_local_experts,
                             num_experts_per_tok=hf.num_experts_per_tok, activation_function="swiglu", add_bias=False,
                             shared_intermediate_size=shared if shared else None))
        elif is_moe:
            mlps.append(dict(mlp_type="MLP", intermediate_size=hf.shared_intermediate_size, activation_function="swiglu", add_bias=False))
        else:
            mlps.append(dict(mlp_type="MLP", intermediate_size=hf.intermediate_size, activation_function="swiglu",
                             add_bias=getattr(hf, "mlp_bias", False)))
    granite = hf.model_type != "llama"
    rope_theta = getattr(hf, "rope_theta", None)
    if rope_theta is None and getattr(hf, "rope_parameters", None):
        rope_theta = hf.rope_parameters.get("rope_theta", 10000)
    position = getattr(hf, "position_embedding_type", "rope") if hf.model_type == "granitemoehybrid" else "rope"
    extra = {}
    if position == "rope" and "mamba2" in kinds:
        extra["rope_dim"] = hf.hidden_size // hf.num_attention_heads
    return GPTBaseConfig(
        vocab_size=hf.vocab_size, max_position_embeddings=hf.max_position_embeddings, hidden_size=hf.hidden_size, num_layers=n,
        normalization_function="rmsnorm", layer_norm_epsilon=hf.rms_norm_eps, initializer_range=hf.initializer_range,
        use_cache=hf.use_cache, position_embedding_type=position, rope_theta=rope_theta or 10000,
        tie_word_embeddings=hf.tie_word_embeddings, bos_token_id=hf.bos_token_id, eos_token_id=hf.eos_token_id, pad_token_id=hf.pad_token_id,
        m_emb=getattr(hf, "embedding_multiplier", None) if granite else None,
        m_residual=getattr(hf, "residual_multiplier", None) if granite else None,
        m_width=getattr(hf, "logits_scaling", None) if granite else None,
        router_aux_loss_coef=getattr(hf, "router_aux_loss_coef", 0.001),
        sequence_mixer_blocks=mixers, mlp_blocks=mlps, **extra)


_ARCHITECTURES = {"llama": "LlamaForCausalLM", "granite": "GraniteForCausalLM", "granitemoe": "GraniteMoeForCausalLM",
                  "granitemoeshared": "GraniteMoeSharedForCausalLM", "granitemoehybrid": "GraniteMoeHybridForCausalLM",
                  "gpt_bigcode": "GPTBigCodeForCausalLM"}


def _export_config(config: GPTBaseConfig, model_type: str):
    from transformers import CONFIG_MAPPING

    if model_type == "gpt_bigcode":
        attn = config.sequence_mixer_blocks[0]
        mlp = config.mlp_blocks[0]
        assert config.normalization_function == "layernorm" and config.position_embedding_type == "learned_absolute"
        assert attn.num_key_value_heads in (1, attn.num_attention_heads)
        return CONFIG_MAPPING["gpt_bigcode"](
            vocab_size=config.vocab_size, n_positions=config.max_position_embeddings, n_embd=config.hidden_size,
            n_layer=config.num_layers, n_head=attn.num_attention_heads, n_inner=mlp.intermediate_size,
            activation_function=mlp.activation_function, resid_pdrop=attn.dropout, embd_pdrop=config.embedding_dropout,
            attn_pdrop=attn.softmax_dropout, layer_norm_epsilon=config.layer_norm_epsilon, initializer_range=config.initializer_range,
            scale_attn_weights=attn.attention_multiplier is None, use_cache=config.use_cache, multi_query=attn.num_key_value_heads == 1,
            tie_word_embeddings=True, bos_token_id=config.bos_token_id, eos_token_id=config.eos_token_id, pad_token_id=config.pad_token_id,
            architectures=[_ARCHITECTURES["gpt_bigcode"]])

    assert config.normalization_function == "rmsnorm"
    attn_blocks = [b for b in config.sequence_mixer_blocks if b.sequence_mixer_type == "softmax_attention"]
    attn = attn_blocks[0]
    mlp = config.mlp_blocks[0]
    kwargs = dict(
        vocab_size=config.vocab_size, max_position_embeddings=config.max_position_embeddings, hidden_size=config.hidden_size,
        num_hidden_layers=config.num_layers, num_attention_heads=attn.num_attention_heads, num_key_value_heads=attn.num_key_value_heads,
        hidden_act="silu", rms_norm_eps=config.layer_norm_epsilon, use_cache=config.use_cache, attention_bias=attn.add_bias,
        tie_word_embeddings=config.tie_word_embeddings, initializer_range=config.initializer_range, rope_theta=config.rope_theta,
        attention_dropout=attn.softmax_dropout, bos_token_id=config.bos_token_id, eos_token_id=config.eos_token_id,
        pad_token_id=config.pad_token_id)
    if model_type != "llama":
        kwargs.update(embedding_multiplier=config.m_emb or 1.0, residual_multiplier=config.m_residual or 1.0,
                      logits_scaling=config.m_width or 1.0,
                      attention_multiplier=attn.attention_multiplier if attn.attention_multiplier is not None else
                      (config.hidden_size // attn.num_attention_heads) ** -0.5)
    if model_type in ("llama", "granite"):
        assert mlp.mlp_type == "MLP" and mlp.activation_function == "swiglu"
        kwargs.update(intermediate_size=mlp.intermediate_size, mlp_bias=mlp.add_bias)
    else:
        moe = next(b for b in config.mlp_blocks if b.mlp_type == "MoE")
        kwargs.update(intermediate_size=moe.intermediate_size, num_local_experts=moe.num_experts,
                      num_experts_per_tok=moe.num_experts_per_tok, router_aux_loss_coef=config.router_aux_loss_coef)
        if model_type in ("granitemoeshared", "granitemoehybrid"):
            kwargs["shared_intermediate_size"] = moe.shared_intermediate_size or 0
        if model_type == "granitemoehybrid":
            kinds = ["mamba" if b.sequence_mixer_type == "mamba2" else "attention" for b in config.sequence_mixer_blocks]
            kwargs.update(layer_types=kinds, position_embedding_type=config.position_embedding_type)
            mamba = next((b for b in config.sequence_mixer_blocks if b.sequence_mixer_type == "mamba2"), None)
            if mamba is not None:
                kwargs.update(mamba_n_heads=mamba.num_heads, mamba_d_state=mamba.state_size, mamba_n_groups=mamba.num_groups,
                              mamba_expand=mamba.intermediate_size // config.hidden_size, mamba_d_conv=mamba.conv_kernel_size,
                              mamba_chunk_size=mamba.chunk_size, mamba_conv_bias=mamba.use_conv_bias, mamba_proj_bias=mamba.add_bias,
                              mamba_d_head=mamba.intermediate_size // mamba.num_heads)
            # carried along as in the reference's export of this family
            kwargs.update(normalization_function=config.normalization_function, init_method=config.init_method)
    # serving stacks choose the model class by this key
    return CONFIG_MAPPING[model_type](architectures=[_ARCHITECTURES[model_type]], **kwargs)


# ----------------------------------------------------------------------------------------------------------------------
# tensor re-layout
_MAMBA_KEYS = ("dt_bias", "A_log", "D", "conv1d.weight", "conv1d.bias", "in_proj.weight", "in_proj.bias", "norm.weight",
               "out_proj.weight", "out_proj.bias")


def _swap_halves(t: torch.Tensor, dim: int) -> torch.Tensor:
    a, b = t.chunk(2, dim=dim)
    return torch.cat([b, a], dim=dim)


def _import_state_dict(config: GPTBaseConfig, hf_type: str, get, has) -> dict[str, torch.Tensor]:
    out = {}
    if hf_type == "gpt_bigcode":
        for name in ("wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias"):
            out[f"transformer.{name}"] = get(f"transformer.{name}")
        for i in range(config.num_layers):
            src, dst = f"transformer.h.{i}.", f"transformer.h.{i}."
            for s in ("weight", "bias"):
                for ln in ("ln_1", "ln_2"):
                    out[f"{dst}{ln}.{s}"] = get(f"{src}{ln}.{s}")
                # same fused layout on both sides: [Q; k; v] for multi-query, [q_h | k_h | v_h] per head otherwise
                out[f"{dst}sequence_mixer.c_attn.{s}"] = get(f"{src}attn.c_attn.{s}")
                out[f"{dst}sequence_mixer.c_proj.{s}"] = get(f"{src}attn.c_proj.{s}")
                out[f"{dst}mlp_block.c_fc.{s}"] = get(f"{src}mlp.c_fc.{s}")
                out[f"{dst}mlp_block.c_proj.{s}"] = get(f"{src}mlp.c_proj.{s}")
        return out

    out["transformer.wte.weight"] = get("model.embed_tokens.weight")
    out["transformer.ln_f.weight"] = get("model.norm.weight")
    if not config.tie_word_embeddings:
        out["lm_head.weight"] = get("lm_head.weight")
    heads_dim = None
    for i in range(config.num_layers):
        src, dst = f"model.layers.{i}.", f"transformer.h.{i}."
        out[f"{dst}ln_1.weight"] = get(f"{src}input_layernorm.weight")
        out[f"{dst}ln_2.weight"] = get(f"{src}post_attention_layernorm.weight")
        mixer = config.sequence_mixer_blocks[i]
        if mixer.sequence_mixer_type == "mamba2":
            for key in _MAMBA_KEYS:
                if has(f"{src}mamba.{key}"):
                    out[f"{dst}sequence_mixer.{key}"] = get(f"{src}mamba.{key}")
        else:
            heads, kv = mixer.num_attention_heads, mixer.num_key_value_heads
            heads_dim = config.hidden_size // heads
            for s in ("weight", "bias"):
                if not has(f"{src}self_attn.q_proj.{s}"):
                    continue
                out[f"{dst}sequence_mixer.c_attn.{s}"] = interleave_query_key_value_tensor_for_attention(
                    get(f"{src}self_attn.q_proj.{s}"), get(f"{src}self_attn.k_proj.{s}"), get(f"{src}self_attn.v_proj.{s}"), heads, kv, heads_dim)
                out[f"{dst}sequence_mixer.c_proj.{s}"] = get(f"{src}self_attn.o_proj.{s}")
        mlp = config.mlp_blocks[i]
        if mlp.mlp_type == "MoE":
            out[f"{dst}mlp_block.gate.weight"] = get(f"{src}block_sparse_moe.router.layer.weight")
            out[f"{dst}mlp_block.c_fc.weight"] = _swap_halves(get(f"{src}block_sparse_moe.input_linear.weight"), dim=1)
            out[f"{dst}mlp_block.c_proj.weight"] = get(f"{src}block_sparse_moe.output_linear.weight")
            if mlp.shared_intermediate_size is not None:
                out[f"{dst}mlp_block.c_fc_shared.weight"] = _swap_halves(get(f"{src}shared_mlp.input_linear.weight"), dim=0)
                out[f"{dst}mlp_block.c_proj_shared.weight"] = get(f"{src}shared_mlp.output_linear.weight")
        elif hf_type in ("granitemoe", "granitemoeshared", "granitemoehybrid"):
            out[f"{dst}mlp_block.c_fc.weight"] = _swap_halves(get(f"{src}shared_mlp.input_linear.weight"), dim=0)
            out[f"{dst}mlp_block.c_proj.weight"] = get(f"{src}shared_mlp.output_linear.weight")
        else:
            for s in ("weight", "bias"):
                if not has(f"{src}mlp.up_proj.{s}"):
                    continue
                out[f"{dst}mlp_block.c_fc.{s}"] = torch.cat([get(f"{src}mlp.up_proj.{s}"), get(f"{src}mlp.gate_proj.{s}")])
                out[f"{dst}mlp_block.c_proj.{s}"] = get(f"{src}mlp.down_proj.{s}")
    return out


def _export_state_dict(config: GPTBaseConfig, hf_type: str, get, has) -> dict[str, torch.Tensor]:
    out = {}
    if hf_type == "gpt_bigcode":
        for name in ("wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias"):
            out[f"transformer.{name}"] = get(f"transformer.{name}")
        for i in range(config.num_layers):
            p = f"transformer.h.{i}."
            for s in ("weight", "bias"):
                for ln in ("ln_1", "ln_2"):
                    out[f"{p}{ln}.{s}"] = get(f"{p}{ln}.{s}")
                out[f"{p}attn.c_attn.{s}"] = get(f"{p}sequence_mixer.c_attn.{s}")
                out[f"{p}attn.c_proj.{s}"] = get(f"{p}sequence_mixer.c_proj.{s}")
                out[f"{p}mlp.c_fc.{s}"] = get(f"{p}mlp_block.c_fc.{s}")
                out[f"{p}mlp.c_proj.{s}"] = get(f"{p}mlp_block.c_proj.{s}")
        return out

    out["model.embed_tokens.weight"] = get("transformer.wte.weight")
    out["model.norm.weight"] = get("transformer.ln_f.weight")
    if not config.tie_word_embeddings:
        out["lm_head.weight"] = get("lm_head.weight")
    for i in range(config.num_layers):
        src, dst = f"transformer.h.{i}.", f"model.layers.{i}."
        out[f"{dst}input_layernorm.weight"] = get(f"{src}ln_1.weight")
        out[f"{dst}post_attention_layernorm.weight"] = get(f"{src}ln_2.weight")
        mixer = config.sequence_mixer_blocks[i]
        if mixer.sequence_mixer_type == "mamba2":
            for key in _MAMBA_KEYS:
                if has(f"{src}sequence_mixer.{key}"):
                    out[f"{dst}mamba.{key}"] = get(f"{src}sequence_mixer.{key}")
        else:
            heads, kv = mixer.num_attention_heads, mixer.num_key_value_heads
            for s in ("weight", "bias"):
                if not has(f"{src}sequence_mixer.c_attn.{s}"):
                    continue
                q, k, v = split_query_key_value_tensor_for_attention(get(f"{src}sequence_mixer.c_attn.{s}"), heads, kv,
                                                                     config.hidden_size // heads)
                out[f"{dst}self_attn.q_proj.{s}"], out[f"{dst}self_attn.k_proj.{s}"], out[f"{dst}self_attn.v_proj.{s}"] = q, k, v
                out[f"{dst}self_attn.o_proj.{s}"] = get(f"{src}sequence_mixer.c_proj.{s}")
        mlp = config.mlp_blocks[i]
        if mlp.mlp_type == "MoE":
            out[f"{dst}block_sparse_moe.router.layer.weight"] = get(f"{src}mlp_block.gate.weight")
            out[f"{dst}block_sparse_moe.input_linear.weight"] = _swap_halves(get(f"{src}mlp_block.c_fc.weight"), dim=1)
            out[f"{dst}block_sparse_moe.output_linear.weight"] = get(f"{src}mlp_block.c_proj.weight")
            if mlp.shared_intermediate_size is not None:
                out[f"{dst}shared_mlp.input_linear.weight"] = _swap_halves(get(f"{src}mlp_block.c_fc_shared.weight"), dim=0)
                out[f"{dst}shared_mlp.output_linear.weight"] = get(f"{src}mlp_block.c_proj_shared.weight")
        elif hf_type in ("granitemoe", "granitemoeshared", "granitemoehybrid"):
            out[f"{dst}shared_mlp.input_linear.weight"] = _swap_halves(get(f"{src}mlp_block.c_fc.weight"), dim=0)
            out[f"{dst}shared_mlp.output_linear.weight"] = get(f"{src}mlp_block.c_proj.weight")
        else:
            for s in ("weight", "bias"):
                if not has(f"{src}mlp_block.c_fc.{s}"):
                    continue
                up, gate = get(f"{src}mlp_block.c_fc.{s}").chunk(2)
                out[f"{dst}mlp.up_proj.{s}"], out[f"{dst}mlp.gate_proj.{s}"] = up, gate
                out[f"{dst}mlp.down_proj.{s}"] = get(f"{src}mlp_block.c_proj.{s}")
    return out


# ----------------------------------------------------------------------------------------------------------------------
def import_from_huggingface(pretrained_model_name_or_path: str, save_path: str) -> None:
    """Read an HF checkpoint (local directory or hub name) and write it in this engine's format."""
    hf_config, tokenizer, weights_path = download_repo(pretrained_model_name_or_path)
    config = _import_config(hf_config)
    manager = SafeTensorsWeightsManager(weights_path)
    state = _import_state_dict(config, hf_config.model_type, manager.get_tensor, manager.has_tensor)
    os.makedirs(save_path, exist_ok=True)
    SafeTensorsWeightsManager.save_state_dict(state, save_path)
    config.save_pretrained(save_path)
    if tokenizer is not None:
        tokenizer.save_pretrained(save_path, legacy_format=False)


def export_to_huggingface(pretrained_model_name_or_path: str, save_path: str, model_type: str) -> None:
    """Write a checkpoint of this engine as the named HF architecture."""
    config, tokenizer, weights_path = download_repo(pretrained_model_name_or_path)
    if not isinstance(config, GPTBaseConfig):
        config = GPTBaseConfig.from_pretrained(pretrained_model_name_or_path)
    hf_config = _export_config(config, model_type)
    manager = SafeTensorsWeightsManager(weights_path)
    state = _export_state_dict(config, model_type, manager.get_tensor, manager.has_tensor)
    os.makedirs(save_path, exist_ok=True)
    SafeTensorsWeightsManager.save_state_dict(state, save_path)
    hf_config.save_pretrained(save_path)
    if tokenizer is not None:
        tokenizer.save_pretrained(save_path, legacy_format=False)


def _family_entry_points() -> None:
    """``import_from_huggingface_<family>`` / ``export_to_huggingface_<family>`` for every supported architecture, the names
    the reference exports (lm_engine/hf_models/model_conversion/__init__.py): the import reads the architecture from the
    checkpoint and refuses another one than the name says, the export fixes the target architecture."""

    def importer(family: str):
        def import_one(pretrained_model_name_or_path: str, save_path: str) -> None:
            hf_config, _, _ = download_repo(pretrained_model_name_or_path)
            expected = "gpt_bigcode" if family == "bigcode" else family
            if hf_config.model_type != expected:
                raise ValueError(f"the checkpoint is a {hf_config.model_type} model, not {expected}")
            import_from_huggingface(pretrained_model_name_or_path, save_path)

        import_one.__name__ = import_one.__qualname__ = f"import_from_huggingface_{family}"
        return import_one

    def exporter(family: str):
        def export_one(pretrained_model_name_or_path: str, save_path: str) -> None:
            export_to_huggingface(pretrained_model_name_or_path, save_path, "gpt_bigcode" if family == "bigcode" else family)

        export_one.__name__ = export_one.__qualname__ = f"export_to_huggingface_{family}"
        return export_one

    for family in ("bigcode",) + _LLAMA_LIKE:
        globals()[f"import_from_huggingface_{family}"] = importer(family)
        globals()[f"export_to_huggingface_{family}"] = exporter(family)


_family_entry_points()

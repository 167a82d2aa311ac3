"""Model configuration: one ``CommonConfig`` with per-layer typed block descriptions.

Parity: lm_engine/hf_models/config/__init__.py:78-232, config/mlp.py:10-28, config/sequence_mixer.py:10-103.
``sequence_mixer_blocks[i]`` and ``mlp_blocks[i]`` describe layer ``i``; they are given as dicts and held as strict
pydantic objects, and serialise back to dicts. Legacy flat arguments (``n_head``, ``num_experts`` ...) are rejected.
A stray ``attention_head_type`` key inside an attention block (present in configs shipped by the reference) is
accepted and ignored: the head layout follows from ``num_attention_heads`` / ``num_key_value_heads``.
"""

from __future__ import annotations

import copy
import inspect
import warnings
from typing import Any

from transformers import PretrainedConfig

from ..utils import BaseArgs, divide_if_divisible


# ----------------------------------------------------------------------------- sequence mixers
class _SoftmaxAttentionArgs(BaseArgs):
    sequence_mixer_type: str = "softmax_attention"
    num_attention_heads: int = 12
    num_key_value_heads: int = 1
    softmax_dropout: float = 0
    dropout: float = 0
    add_bias: bool = True
    attention_multiplier: float | None = None


class _MultiHeadLatentAttentionArgs(BaseArgs):
    sequence_mixer_type: str = "multihead_latent_attention"
    num_attention_heads: int | None = None
    softmax_dropout: float = 0
    dropout: float = 0
    add_bias: bool = True
    attention_multiplier: float | None = None
    query_compression_size: int | None = None
    key_value_compression_size: int | None = None
    head_dim: int | None = None
    normalization_function: str = "layernorm"

    def model_post_init(self, __context: Any) -> None:
        for name in ("num_attention_heads", "query_compression_size", "key_value_compression_size", "head_dim"):
            if getattr(self, name) is None:
                raise ValueError(f"multihead_latent_attention needs {name}")


class _StickbreakingAttentionArgs(BaseArgs):
    sequence_mixer_type: str = "stickbreaking_attention"
    num_attention_heads: int = 12
    num_key_value_heads: int = 1
    dropout: float = 0
    add_bias: bool = True
    attention_multiplier: float | None = None


class _Mamba2Args(BaseArgs):
    sequence_mixer_type: str = "mamba2"
    state_size: int = 128
    intermediate_size: int
    num_heads: int = 128
    conv_kernel_size: int = 4
    time_step_limit: tuple[float, float] = (0, float("inf"))
    add_bias: bool = True
    use_conv_bias: bool = True
    activation_function: str = "silu"
    num_groups: int = 8
    chunk_size: int = 256


class _GRUArgs(BaseArgs):
    sequence_mixer_type: str = "gru"
    state_size: int = 2048
    num_heads: int = 128
    add_bias: bool = True
    normalization_function: str | None = None
    gradient_clipping: float | None = None


class _RNNArgs(_GRUArgs):
    sequence_mixer_type: str = "rnn"


class _CausalConvolution(BaseArgs):
    sequence_mixer_type: str = "causal_convolution"
    activation_function: str = "silu"
    in_channels: int
    out_channels: int
    kernel_size: int
    num_groups: int
    add_bias: bool = False


# ----------------------------------------------------------------------------- MLP blocks
class _MLPArgs(BaseArgs):
    mlp_type: str = "MLP"
    intermediate_size: int
    activation_function: str = "gelu_pytorch_tanh"
    dropout: float = 0
    add_bias: bool = True


class _MoEArgs(_MLPArgs):
    mlp_type: str = "MoE"
    shared_intermediate_size: int | None = None
    num_experts: int = 8
    num_experts_per_tok: int = 2


_MIXER_CLASSES: dict[str, type[BaseArgs]] = {
    "causal_convolution": _CausalConvolution,
    "gru": _GRUArgs,
    "mamba2": _Mamba2Args,
    "multihead_latent_attention": _MultiHeadLatentAttentionArgs,
    "rnn": _RNNArgs,
    "stickbreaking_attention": _StickbreakingAttentionArgs,
    "softmax_attention": _SoftmaxAttentionArgs,
}
_MLP_CLASSES: dict[str, type[BaseArgs]] = {"MLP": _MLPArgs, "MoE": _MoEArgs}

# flat arguments of older config generations; their presence is an error
_LEGACY_FLAT_ARGS = (
    "activation_function attn_pdrop embd_pdrop resid_pdrop intermediate_size shared_intermediate_size num_experts "
    "num_experts_per_tok add_bias attention_blocks num_key_value_heads attention_head_type attention_multiplier "
    "n_embd n_head n_inner n_layer n_positions scale_attn_weights num_attention_heads"
).split()


def _as_plain(blocks: list) -> list[dict]:
    return [b.to_dict() if isinstance(b, BaseArgs) else copy.deepcopy(b) for b in blocks]


def _build_mixer_block(raw: dict | BaseArgs, hidden_size: int) -> BaseArgs:
    if isinstance(raw, BaseArgs):
        return raw
    raw = dict(raw)
    kind = raw.pop("sequence_mixer_type", "softmax_attention")
    if kind not in _MIXER_CLASSES:
        raise ValueError(f"unknown sequence_mixer_type ({kind})")
    if "attention_head_type" in raw:
        warnings.warn("ignoring legacy key `attention_head_type` in a sequence mixer block", stacklevel=3)
        raw.pop("attention_head_type")
    if kind == "mamba2":
        raw.setdefault("intermediate_size", 2 * hidden_size)
    return _MIXER_CLASSES[kind](sequence_mixer_type=kind, **raw)


def _build_mlp_block(raw: dict | BaseArgs, hidden_size: int) -> BaseArgs:
    if isinstance(raw, BaseArgs):
        return raw
    raw = dict(raw)
    kind = raw.pop("mlp_type", "MLP")
    if kind not in _MLP_CLASSES:
        raise ValueError(f"unknown mlp_type ({kind})")
    raw.setdefault("intermediate_size", 4 * hidden_size)
    return _MLP_CLASSES[kind](mlp_type=kind, **raw)


class CommonConfig(PretrainedConfig):
    keys_to_ignore_at_inference = ["past_key_values"]

    def __init__(
        self,
        vocab_size: int = 50304,
        max_position_embeddings: int = 1024,
        hidden_size: int = 768,
        num_layers: int = 12,
        embedding_dropout: float = 0,
        normalization_function: str = "layernorm",
        layer_norm_epsilon: float = 1e-5,
        initializer_range: float = 0.02,
        use_cache: bool = True,
        bos_token_id: int = 50256,
        eos_token_id: int = 50256,
        pad_token_id: int = 50256,
        position_embedding_type: str = "learned_absolute",
        rope_theta: int = 10000,
        rope_scaling: dict | None = None,
        m_emb: float | None = None,
        m_width: float | None = None,
        m_residual: float | None = None,
        init_method: str = "normal",
        sequence_mixer_blocks: list[dict] | None = None,
        mlp_blocks: list[dict] | None = None,
        router_aux_loss_coef: float = 0.001,
        tie_word_embeddings: bool = True,
        rope_dim: int | None = None,
        **kwargs,
    ) -> None:
        if init_method not in ("normal", "mup"):
            raise ValueError(f"unexpected init_method ({init_method})")
        if position_embedding_type not in ("rope", "learned_absolute", "nope"):
            raise ValueError(f"unexpected position_embedding_type ({position_embedding_type})")
        for name in _LEGACY_FLAT_ARGS:
            if name in kwargs:
                raise ValueError(f"found legacy flat argument ({name}); describe layers in the per-layer block lists")

        self.vocab_size = vocab_size
        self.max_position_embeddings = max_position_embeddings
        self.hidden_size = hidden_size
        self.num_layers = num_layers
        self.embedding_dropout = embedding_dropout
        self.normalization_function = normalization_function
        self.layer_norm_epsilon = layer_norm_epsilon
        self.initializer_range = initializer_range
        self.use_cache = use_cache
        self.position_embedding_type = position_embedding_type
        self.rope_theta = rope_theta
        self.rope_scaling = rope_scaling
        self.m_emb = m_emb
        self.m_width = m_width
        self.m_residual = m_residual
        self.init_method = init_method
        self.router_aux_loss_coef = router_aux_loss_coef

        mixers = sequence_mixer_blocks if sequence_mixer_blocks is not None else [{} for _ in range(num_layers)]
        mlps = mlp_blocks if mlp_blocks is not None else [{} for _ in range(num_layers)]
        if len(mixers) != num_layers or len(mlps) != num_layers:
            raise ValueError("sequence_mixer_blocks and mlp_blocks need one entry per layer")
        self.sequence_mixer_blocks = [_build_mixer_block(b, hidden_size) for b in mixers]
        self.mlp_blocks = [_build_mlp_block(b, hidden_size) for b in mlps]

        self.rope_dim = rope_dim
        if rope_dim is None and position_embedding_type == "rope":
            kinds = {b.sequence_mixer_type for b in self.sequence_mixer_blocks}
            if kinds != {"softmax_attention"}:
                raise ValueError("rope_dim must be given when not every layer is softmax attention")
            heads = self.check_equal_for_all_and_get_value("sequence_mixer_blocks", "num_attention_heads")
            self.rope_dim = divide_if_divisible(hidden_size, heads, "hidden_size must be divisible by the head count")

        super().__init__(
            bos_token_id=bos_token_id,
            eos_token_id=eos_token_id,
            pad_token_id=pad_token_id,
            tie_word_embeddings=tie_word_embeddings,
            **kwargs,
        )
        # make sure the token ids / tie flag exist as plain attributes on every transformers version
        for name, value in (
            ("bos_token_id", bos_token_id),
            ("eos_token_id", eos_token_id),
            ("pad_token_id", pad_token_id),
            ("tie_word_embeddings", tie_word_embeddings),
        ):
            if getattr(self, name, None) is None and value is not None:
                setattr(self, name, value)

    # ------------------------------------------------------------------ serialisation
    def to_dict(self) -> dict:
        typed = (self.sequence_mixer_blocks, self.mlp_blocks)
        self.sequence_mixer_blocks, self.mlp_blocks = _as_plain(typed[0]), _as_plain(typed[1])
        try:
            out = super().to_dict()
        finally:
            self.sequence_mixer_blocks, self.mlp_blocks = typed
        return out

    def to_diff_dict(self) -> dict:
        """What ``config.json`` holds: every key of this model family (also those at their defaults, so that the file reads
        on its own) plus the generic transformers keys that differ from their defaults."""
        typed = (self.sequence_mixer_blocks, self.mlp_blocks)
        self.sequence_mixer_blocks, self.mlp_blocks = _as_plain(typed[0]), _as_plain(typed[1])
        try:
            out = super().to_diff_dict()
        finally:
            self.sequence_mixer_blocks, self.mlp_blocks = typed
        full = self.to_dict()
        for key in inspect.signature(CommonConfig.__init__).parameters:
            if key in full:
                out[key] = full[key]
        for key in set(full) - set(PretrainedConfig().to_dict()):  # keys of a subclass (sharing pattern and the like)
            out.setdefault(key, full[key])
        return out

    def __deepcopy__(self, memo):
        return type(self).from_dict(copy.deepcopy(self.to_dict(), memo))

    # ------------------------------------------------------------------ helpers
    def yarn_scaling(self) -> dict | None:
        """``{"factor", "original_max_position_embeddings"}`` when YaRN scaling is configured, else None. (Newer
        transformers versions rewrite ``rope_scaling`` into a normalised dict that always exists.)"""
        scaling = getattr(self, "rope_scaling", None)
        if not scaling or "factor" not in scaling:
            return None
        return {
            "factor": scaling["factor"],
            "original_max_position_embeddings": scaling.get("original_max_position_embeddings", self.max_position_embeddings),
        }

    def check_equal_for_all_and_get_value(
        self, key: str, key_block: str, expected_value: Any | None = None, sequence_mixer_type: str | None = None
    ) -> Any:
        """Value of ``key_block`` shared by all blocks of list ``key`` (optionally only blocks of one mixer type)."""
        blocks = list(getattr(self, key))
        if sequence_mixer_type is not None:
            blocks = [b for b in blocks if _get(b, "sequence_mixer_type") == sequence_mixer_type]
        values = [_get(b, key_block) for b in blocks]
        if any(v != values[0] for v in values):
            raise ValueError(f"{key}.{key_block} differs across layers: {values}")
        if expected_value is not None and values[0] != expected_value:
            raise ValueError(f"{key}.{key_block} is {values[0]}, expected {expected_value}")
        return values[0]


def _get(block, name):
    return block.get(name) if isinstance(block, dict) else getattr(block, name)


class GPTBaseConfig(CommonConfig):
    model_type = "gpt_base"

    def __init__(self, **kwargs) -> None:
        super().__init__(**kwargs)


class PaLMConfig(CommonConfig):
    model_type = "palm"

    def __init__(self, **kwargs) -> None:
        super().__init__(**kwargs)


class LadderResidualConfig(CommonConfig):
    model_type = "ladder_residual"

    def __init__(self, **kwargs) -> None:
        super().__init__(**kwargs)


class GPTCrossLayerConfig(CommonConfig):
    """Adds ``sharing_pattern``: ``sharing_pattern[i] = j`` makes layer ``i`` reuse the keys/values of layer ``j``
    (parity: lm_engine/hf_models/models/gpt_crosslayer/config.py:10-48)."""

    model_type = "gpt_crosslayer"

    def __init__(self, sharing_pattern: list[int] | None = None, **kwargs) -> None:
        super().__init__(**kwargs)
        if sharing_pattern is None:
            sharing_pattern = list(range(self.num_layers))
        if len(sharing_pattern) != self.num_layers:
            raise ValueError("sharing_pattern needs one entry per layer")
        for i, parent in enumerate(sharing_pattern):
            if parent > i or parent < 0:
                raise ValueError("a layer can only share with itself or an earlier layer")
            if sharing_pattern[parent] != parent:
                raise ValueError("a layer can only share with a layer that owns its keys/values")
            mine, theirs = self.sequence_mixer_blocks[i], self.sequence_mixer_blocks[parent]
            if getattr(mine, "sequence_mixer_type", None) != getattr(theirs, "sequence_mixer_type", None):
                # rotary embeddings are applied to the keys of softmax layers only: a stick-breaking layer cannot read them
                raise ValueError("layers that share keys/values need the same sequence_mixer_type")
        self.sharing_pattern = sharing_pattern


class DesyncResidualConfig(CommonConfig):
    """Single-process simulation of tensor parallel training with skipped all-reduces
    (parity: lm_engine/hf_models/models/desync_residual/config.py)."""

    model_type = "desync_residual"

    def __init__(
        self,
        pretraining_tensor_parallel_size: int = 1,
        reduce_pattern: list[dict] | None = None,
        **kwargs,
    ) -> None:
        super().__init__(**kwargs)
        self.pretraining_tensor_parallel_size = pretraining_tensor_parallel_size
        if reduce_pattern is None:
            reduce_pattern = [{"attention": True, "mlp": True} for _ in range(self.num_layers)]
        self.reduce_pattern = reduce_pattern

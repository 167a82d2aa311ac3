"""Generation cache holding one state per layer: concatenating key/value cache for attention layers, a single
recurrent state for RNN/GRU layers and a (conv window, ssm state) pair for Mamba-2 layers.

Parity: lm_engine/hf_models/cache/{__init__.py:25-56, softmax_attention.py, rnn.py, mamba2.py}.
"""

from __future__ import annotations

import torch


class _KVState:
    def __init__(self) -> None:
        self.key: torch.Tensor | None = None
        self.value: torch.Tensor | None = None
        self.seen_tokens = 0

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor | None = None, sequence_length_dimension: int = -2):
        self.seen_tokens += key_states.shape[sequence_length_dimension]
        if self.key is None:
            self.key, self.value = key_states, value_states
        else:
            self.key = torch.cat([self.key, key_states], dim=sequence_length_dimension)
            if value_states is not None:
                self.value = torch.cat([self.value, value_states], dim=sequence_length_dimension)
        return self.key, self.value

    def get(self):
        return self.key, self.value

    def reorder(self, beam_idx: torch.Tensor) -> None:
        if self.key is not None:
            self.key = self.key.index_select(0, beam_idx.to(self.key.device))
        if self.value is not None:
            self.value = self.value.index_select(0, beam_idx.to(self.value.device))


class _RecurrentState:
    def __init__(self) -> None:
        self.state: torch.Tensor | None = None
        self.seen_tokens = 0

    def update(self, state: torch.Tensor, num_tokens_added: int = 1):
        self.seen_tokens += num_tokens_added
        self.state = state
        return state

    def get(self):
        return self.state

    def reorder(self, beam_idx: torch.Tensor) -> None:
        if self.state is not None:
            self.state = self.state.index_select(0, beam_idx.to(self.state.device))


class _Mamba2State:
    def __init__(self) -> None:
        self.conv_state: torch.Tensor | None = None
        self.ssm_state: torch.Tensor | None = None
        self.seen_tokens = 0

    def update(self, conv_state: torch.Tensor | None = None, ssm_state: torch.Tensor | None = None, num_tokens_added: int = 0):
        self.seen_tokens += num_tokens_added
        if conv_state is not None:
            self.conv_state = conv_state
        if ssm_state is not None:
            self.ssm_state = ssm_state
        return self.conv_state, self.ssm_state

    def get(self):
        return self.conv_state, self.ssm_state

    def reorder(self, beam_idx: torch.Tensor) -> None:
        for name in ("conv_state", "ssm_state"):
            t = getattr(self, name)
            if t is not None:
                setattr(self, name, t.index_select(0, beam_idx.to(t.device)))


_STATE_OF_MIXER = {
    "softmax_attention": _KVState,
    "stickbreaking_attention": _KVState,
    "multihead_latent_attention": _KVState,
    "causal_convolution": _RecurrentState,
    "gru": _RecurrentState,
    "rnn": _RecurrentState,
    "mamba2": _Mamba2State,
}


class GenerationCache:
    def __init__(self, config) -> None:
        self._seen_tokens = 0
        self.cache = [_STATE_OF_MIXER[block.sequence_mixer_type]() for block in config.sequence_mixer_blocks]

    def __len__(self) -> int:
        return len(self.cache)

    def update(self, *, layer_idx: int, **kwargs):
        return self.cache[layer_idx].update(**kwargs)

    def get_cache(self, layer_idx: int):
        return self.cache[layer_idx].get()

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.cache[layer_idx].seen_tokens

    def get_max_cache_shape(self):
        return None

    def get_mask_sizes(self, cache_position, layer_idx: int = 0):
        return self.get_seq_length(layer_idx) + cache_position.shape[0], 0

    def reorder_cache(self, beam_idx: torch.Tensor) -> None:
        for state in self.cache:
            state.reorder(beam_idx)

    # some generation utilities probe these
    @property
    def is_compileable(self) -> bool:
        return False

    def crop(self, max_length: int) -> None:
        raise NotImplementedError("cropping is not supported by this cache")

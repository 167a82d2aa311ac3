"""Sharding and unsharding of checkpoints for tensor (and pipeline) parallel models.

Parity: lm_engine/hf_models/models/gpt_base_TP/weights/{shard.py:13-307, unshard.py:12-274, fix.py:11-66} and
lm_engine/hf_models/modeling_utils_TP/TP.py:11-40. One table of rules, keyed by the parameter's name, drives all three
directions: every rule says along which dimension a tensor is split and in how many stacked blocks (a gated ``c_fc`` is
two blocks, ``[up ; gate]``, each split on its own so that every rank's local tensor is again ``[up_r ; gate_r]``).
Reading goes through lazy safetensors slices, so a rank touches only the bytes it keeps.
"""

from __future__ import annotations

import math
import re

import torch

from ..parallel import tensor_parallel as tp
from ..utils import SafeTensorsWeightsManager, divide_if_divisible
from .layers.activations import is_glu

VOCAB_MULTIPLE = 64


def tensor_parallel_split_safetensor_slice(slice_, dim: int, start_end: tuple[int, int] | None = None, rank: int | None = None,
                                           world: int | None = None) -> torch.Tensor:
    """This rank's part of a lazily opened tensor (at most 3-D) along ``dim``; ``start_end`` overrides the even split."""
    shape = slice_.get_shape()
    dim = dim % len(shape)
    if start_end is None:
        world = tp.tp_world() if world is None else world
        rank = tp.tp_rank() if rank is None else rank
        stride = divide_if_divisible(shape[dim], world, f"split dimension ({dim}) is not divisible by the tensor parallel size")
        start_end = (rank * stride, (rank + 1) * stride)
    index = [slice(None)] * len(shape)
    index[dim] = slice(*start_end)
    return slice_[tuple(index)]


def _rule(config, name: str, tp_world: int) -> tuple[str, int, int]:
    """(kind, dim, parts) for a parameter of the unsharded model: kind in {"split", "vocab", "replicate", "mqa"}."""
    if name.endswith(("wte.weight", "lm_head.weight", "wpe.weight")):
        return "vocab", 0, 1  # the position table is a padded, row-sharded embedding as well (as in the reference)
    match = re.search(r"\.h\.(\d+)\.(sequence_mixer|mlp_block)\.(\w+)\.(weight|bias)$", name)
    if match is None:
        return "replicate", 0, 1
    layer, block, module, kind = int(match.group(1)), match.group(2), match.group(3), match.group(4)
    if block == "sequence_mixer":
        mixer = config.sequence_mixer_blocks[layer]
        if module == "c_attn":
            if mixer.num_key_value_heads == 1 and tp_world > 1:
                return "mqa", 0, 1
            return "split", 0, 1
        if module == "c_proj":
            return ("split", 1, 1) if kind == "weight" else ("replicate", 0, 1)
        return "replicate", 0, 1
    mlp = config.mlp_blocks[layer]
    glu = 2 if is_glu(mlp.activation_function) else 1
    experts = mlp.mlp_type == "MoE" and module in ("c_fc", "c_proj")
    if module in ("c_fc", "c_fc_shared"):
        return "split", (1 if experts else 0), glu
    if module in ("c_proj", "c_proj_shared"):
        if kind == "bias":
            return "replicate", 0, 1
        return "split", (2 if experts else 1), 1
    return "replicate", 0, 1  # router


def _padded_vocab(vocab_size: int) -> int:
    return VOCAB_MULTIPLE * math.ceil(vocab_size / VOCAB_MULTIPLE)


def _table_rows(config, name: str) -> int:
    """Rows of an embedding table without its padding."""
    return config.max_position_embeddings if name.endswith("wpe.weight") else config.vocab_size


def _split_blocks(full: torch.Tensor, dim: int, parts: int, rank: int, world: int) -> torch.Tensor:
    blocks = full.chunk(parts, dim=dim)
    return torch.cat([b.chunk(world, dim=dim)[rank] for b in blocks], dim=dim).contiguous()


def _stage_layers(config, num_pipeline_stages: int, pipeline_stage_id: int) -> range:
    per_stage = divide_if_divisible(config.num_layers, num_pipeline_stages, "layers should be divisible by num_pipeline_stages")
    return range(per_stage * pipeline_stage_id, per_stage * (pipeline_stage_id + 1))


def _names_of_stage(config, all_names: list[str], num_pipeline_stages: int, pipeline_stage_id: int) -> list[str]:
    layers = set(_stage_layers(config, num_pipeline_stages, pipeline_stage_id))
    first, last = pipeline_stage_id == 0, pipeline_stage_id == num_pipeline_stages - 1
    keep = []
    for name in all_names:
        match = re.search(r"\.h\.(\d+)\.", name)
        if match is not None:
            if int(match.group(1)) in layers:
                keep.append(name)
        elif ".wte." in name or ".wpe." in name:
            if first or (last and ".wte." in name and config.tie_word_embeddings):
                keep.append(name)
        elif ".ln_f." in name or name.startswith("lm_head."):
            if last:
                keep.append(name)
        else:
            keep.append(name)
    return keep


def shard_tensor(config, name: str, read, shape: tuple[int, ...], rank: int, world: int) -> dict[str, torch.Tensor]:
    """Local tensors made from one full tensor. ``read(index)`` returns ``full[index]`` (so that a lazy slice can serve)."""
    kind, dim, parts = _rule(config, name, world)
    everything = tuple(slice(None) for _ in shape)
    if kind == "replicate" or world == 1 and kind != "vocab":
        return {name: read(everything)}
    if kind == "vocab":
        per_rank = _padded_vocab(shape[0]) // world
        start, end = rank * per_rank, min((rank + 1) * per_rank, shape[0])
        rows = read((slice(start, max(end, start)),) + everything[1:])
        if rows.shape[0] < per_rank:
            rows = torch.cat([rows, rows.new_zeros(per_rank - rows.shape[0], *rows.shape[1:])])
        return {name: rows}
    if kind == "mqa":
        mixer = config.sequence_mixer_blocks[int(re.search(r"\.h\.(\d+)\.", name).group(1))]
        head_dim = config.hidden_size // mixer.num_attention_heads
        q_rows = shape[0] - 2 * head_dim
        stride = q_rows // world
        suffix = name.rsplit(".", 1)[1]
        base = name[: -len(suffix)]  # "...sequence_mixer.c_attn."
        return {base + "q_attn." + suffix: read((slice(rank * stride, (rank + 1) * stride),) + everything[1:]),
                base + "kv_attn." + suffix: read((slice(q_rows, shape[0]),) + everything[1:])}
    block = shape[dim] // parts
    stride = divide_if_divisible(block, world, f"{name}: dimension {dim} is not divisible by the tensor parallel size")
    pieces = []
    for b in range(parts):
        index = list(everything)
        index[dim] = slice(b * block + rank * stride, b * block + (rank + 1) * stride)
        pieces.append(read(tuple(index)))
    return {name: pieces[0] if parts == 1 else torch.cat(pieces, dim=dim)}


def get_gpt_base_model_parallel_state_dict(config, safetensors_weights_manager: SafeTensorsWeightsManager, num_pipeline_stages: int = 1,
                                           pipeline_stage_id: int = 0, rank: int | None = None, world: int | None = None) -> dict[str, torch.Tensor]:
    """State dict of this rank's tensor-parallel, pipeline-stage-local model read from an unsharded checkpoint."""
    rank = tp.tp_rank() if rank is None else rank
    world = tp.tp_world() if world is None else world
    out = {}
    for name in _names_of_stage(config, list(safetensors_weights_manager.keys()), num_pipeline_stages, pipeline_stage_id):
        lazy = safetensors_weights_manager.get_slice(name)
        out.update(shard_tensor(config, name, lambda index, lazy=lazy: lazy[index], tuple(lazy.get_shape()), rank, world))
    return out


def shard_state_dict(config, state_dict: dict[str, torch.Tensor], rank: int, world: int, num_pipeline_stages: int = 1,
                     pipeline_stage_id: int = 0) -> dict[str, torch.Tensor]:
    """Same as :func:`get_gpt_base_model_parallel_state_dict` for tensors already in memory."""
    out = {}
    for name in _names_of_stage(config, list(state_dict), num_pipeline_stages, pipeline_stage_id):
        full = state_dict[name]
        out.update(shard_tensor(config, name, lambda index, full=full: full[index].clone(), tuple(full.shape), rank, world))
    return out


def unshard_tensor_parallel_state_dicts(config, tensor_parallel_state_dicts: list[dict[str, torch.Tensor]], prefix: str = "",
                                        check_correctness: bool = True) -> dict[str, torch.Tensor]:
    """The unsharded state dict from the local state dicts of all tensor-parallel ranks (in rank order). State dicts of
    several pipeline stages can be merged beforehand with ``dict.update``: their keys are disjoint."""
    world = len(tensor_parallel_state_dicts)
    first = tensor_parallel_state_dicts[0]
    out: dict[str, torch.Tensor] = {}
    for key in first:
        name = key[len(prefix):] if prefix and key.startswith(prefix) else key
        pieces = [sd[key] for sd in tensor_parallel_state_dicts]
        if ".q_attn." in name or ".kv_attn." in name:
            if ".kv_attn." in name:
                continue
            suffix = name.rsplit(".", 1)[1]
            kv = [sd[key.replace(".q_attn.", ".kv_attn.")] for sd in tensor_parallel_state_dicts]
            if check_correctness:
                assert all(torch.equal(kv[0], other) for other in kv[1:]), f"{name}: replicated kv_attn differs between ranks"
            out[prefix + name.replace("c_attn.q_attn." + suffix, "c_attn." + suffix)] = torch.cat(pieces + [kv[0]], dim=0)
            continue
        kind, dim, parts = _rule(config, name, world)
        if kind == "replicate":
            if check_correctness:
                assert all(torch.equal(pieces[0], other) for other in pieces[1:]), f"{name}: replicated tensor differs between ranks"
            out[key] = pieces[0]
        elif kind == "vocab":
            out[key] = torch.cat(pieces, dim=0)[: _table_rows(config, name)]
        else:
            blocks = [p.chunk(parts, dim=dim) for p in pieces]
            out[key] = torch.cat([torch.cat([blocks[r][b] for r in range(world)], dim=dim) for b in range(parts)], dim=dim)
    return out


def fix_unsharded_state_dict(config, state_dict: dict[str, torch.Tensor], tensor_parallel_world_size: int, prefix: str = "") -> dict[str, torch.Tensor]:
    """Repairs a state dict that was assembled by plainly concatenating every rank's tensors along their split
    dimension: drops the vocabulary padding, restores ``[up ; gate]`` from ``[up_0 ; gate_0 ; up_1 ; gate_1 ...]`` and
    folds ``q_attn`` / ``kv_attn`` back into ``c_attn``."""
    world = tensor_parallel_world_size
    out = dict(state_dict)
    for key in list(state_dict):
        name = key[len(prefix):] if prefix and key.startswith(prefix) else key
        if ".kv_attn." in name:
            continue
        if ".q_attn." in name:
            suffix = name.rsplit(".", 1)[1]
            kv_key = key.replace(".q_attn.", ".kv_attn.")
            out[key.replace("c_attn.q_attn." + suffix, "c_attn." + suffix)] = torch.cat([state_dict[key], state_dict[kv_key]], dim=0)
            del out[key], out[kv_key]
            continue
        kind, dim, parts = _rule(config, name, world)
        value = state_dict[key]
        if kind == "vocab":
            out[key] = value[: _table_rows(config, name)]
        elif kind == "split" and parts > 1:
            per_rank = value.chunk(world, dim=dim)
            out[key] = torch.cat([torch.cat([p.chunk(parts, dim=dim)[b] for p in per_rank], dim=dim) for b in range(parts)], dim=dim)
    return out

"""Lazy reader over a directory of safetensors shards and a sharded writer with an HF-style index.

Parity: lm_engine/utils/safetensors.py:15-101 (``get_slice``, ``get_tensor``, ``get_shape``, ``has_tensor``,
``state_dict``, ``save_state_dict``, equality of two managers).
"""

from __future__ import annotations

import json
import os

import torch
from safetensors import safe_open
from safetensors.torch import save_file

_INDEX_NAME = "model.safetensors.index.json"


class SafeTensorsWeightsManager:
    def __init__(self, model_path: str) -> None:
        self.model_path = model_path
        self._file_of_tensor: dict[str, str] = {}
        self._handles: dict[str, object] = {}
        for name in sorted(os.listdir(model_path)):
            if not name.endswith(".safetensors"):
                continue
            full = os.path.join(model_path, name)
            with safe_open(full, framework="pt") as handle:
                for key in handle.keys():
                    self._file_of_tensor[key] = full

    def _handle(self, tensor_name: str):
        path = self._file_of_tensor[tensor_name]
        if path not in self._handles:
            self._handles[path] = safe_open(path, framework="pt")
        return self._handles[path]

    def get_slice(self, tensor_name: str):
        return self._handle(tensor_name).get_slice(tensor_name)

    def get_tensor(self, tensor_name: str, dtype: torch.dtype | None = None, device=None) -> torch.Tensor:
        tensor = self._handle(tensor_name).get_tensor(tensor_name)
        if dtype is not None or device is not None:
            tensor = tensor.to(dtype=dtype, device=device)
        return tensor

    def get_shape(self, tensor_name: str) -> tuple[int, ...]:
        return tuple(self.get_slice(tensor_name).get_shape())

    def has_tensor(self, tensor_name: str) -> bool:
        return tensor_name in self._file_of_tensor

    def __len__(self) -> int:
        return len(self._file_of_tensor)

    def __iter__(self):
        return iter(self._file_of_tensor)

    def keys(self):
        return self._file_of_tensor.keys()

    def state_dict(self) -> dict[str, torch.Tensor]:
        return {name: self.get_tensor(name) for name in self._file_of_tensor}

    def __eq__(self, other) -> bool:
        if not isinstance(other, SafeTensorsWeightsManager):
            return False
        if set(self.keys()) != set(other.keys()):
            return False
        return all(self.get_tensor(name).equal(other.get_tensor(name)) for name in self.keys())

    @staticmethod
    def save_state_dict(state_dict: dict[str, torch.Tensor], save_path: str, max_shard_size: int = 5 * 2**30) -> None:
        """Write ``state_dict`` as one or more safetensors files plus ``model.safetensors.index.json``."""
        os.makedirs(save_path, exist_ok=True)
        shards: list[dict[str, torch.Tensor]] = [{}]
        used = 0
        total = 0
        for name, tensor in state_dict.items():
            nbytes = tensor.numel() * tensor.element_size()
            if used > 0 and used + nbytes > max_shard_size:
                shards.append({})
                used = 0
            shards[-1][name] = tensor.detach().contiguous().cpu()
            used += nbytes
            total += nbytes

        if len(shards) == 1:
            save_file(shards[0], os.path.join(save_path, "model.safetensors"), metadata={"format": "pt"})
            return

        weight_map = {}
        for i, shard in enumerate(shards):
            file_name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(shard, os.path.join(save_path, file_name), metadata={"format": "pt"})
            for name in shard:
                weight_map[name] = file_name
        with open(os.path.join(save_path, _INDEX_NAME), "w") as handle:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, handle, indent=2)

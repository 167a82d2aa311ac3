"""Resolve a model name or local path to (config, tokenizer, directory with safetensors weights)."""

from __future__ import annotations

import os

from transformers import AutoConfig, AutoTokenizer


def _try(factory, name: str):
    try:
        return factory(name)
    except Exception:
        return None


def download_repo(repo_name_or_path: str):
    """Parity: lm_engine/utils/hf_hub.py:12-51. Works offline for local directories."""
    config = _try(AutoConfig.from_pretrained, repo_name_or_path)
    tokenizer = _try(AutoTokenizer.from_pretrained, repo_name_or_path)
    if os.path.isdir(repo_name_or_path):
        return config, tokenizer, repo_name_or_path

    from huggingface_hub import snapshot_download

    path = snapshot_download(repo_name_or_path, allow_patterns=["*.safetensors", "*.json"])
    return config, tokenizer, path

"""Command line utilities: parameter calculator, store merge / inspect."""

import json
import sys

import numpy as np

from lm_engine.data.megatron.indexed_dataset import MMapIndexedDatasetBuilder, get_bin_path, get_idx_path
from lm_engine.hf_models import GPTBaseConfig


def _run(module, argv, capsys):
    old = sys.argv
    sys.argv = [module.__name__] + argv
    try:
        module.main()
    finally:
        sys.argv = old
    return capsys.readouterr().out


def test_params_calculator_counts_total_and_active(tmp_path, capsys):
    from lm_engine.cli import params_calculator

    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    moe = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=32, add_bias=False, num_experts=8, num_experts_per_tok=2)
    config = GPTBaseConfig(vocab_size=128, hidden_size=64, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           tie_word_embeddings=False, sequence_mixer_blocks=[attn, attn], mlp_blocks=[moe, moe])
    config.save_pretrained(tmp_path)
    out = json.loads(_run(params_calculator, ["--config", str(tmp_path), "--sequence-length", "128"], capsys))
    experts = 2 * 8 * (2 * 32 * 64 + 64 * 32)
    assert out["total_parameters"] - out["active_parameters"] == experts * 6 // 8
    assert out["tflop_per_step"] > 0


def test_store_merge_and_inspect(tmp_path, capsys):
    from lm_engine.cli import preprocess_data

    prefixes = []
    for i in range(2):
        prefix = str(tmp_path / f"part{i}")
        builder = MMapIndexedDatasetBuilder(get_bin_path(prefix), dtype=np.uint16)
        for j in range(3):
            builder.add_item(np.arange(5 + i + j))
            builder.end_document()
        builder.finalize(get_idx_path(prefix))
        prefixes.append(prefix)
    merged = str(tmp_path / "merged")
    _run(preprocess_data, ["merge", "--input", *prefixes, "--output-prefix", merged], capsys)
    out = _run(preprocess_data, ["inspect", "--path-prefix", merged, "--show", "1"], capsys)
    assert "sequences: 6" in out and "documents: 6" in out and "tokens: 39" in out and "[0, 1, 2, 3, 4]" in out

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


def _tiny_model_with_tokenizer(path: str):
    import torch
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from lm_engine.hf_models import GPTBaseForCausalLM

    words = ["<eos>", "<pad>"] + [f"w{i}" for i in range(62)]
    tokenizer = Tokenizer(models.WordLevel({word: index for index, word in enumerate(words)}, unk_token="w0"))
    tokenizer.pre_tokenizer = pre_tokenizers.Whitespace()
    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=64, add_bias=False)
    torch.manual_seed(0)
    config = GPTBaseConfig(vocab_size=64, hidden_size=32, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           tie_word_embeddings=False, bos_token_id=0, eos_token_id=0, pad_token_id=1,
                           sequence_mixer_blocks=[attn, dict(attn)], mlp_blocks=[mlp, dict(mlp)])
    model = GPTBaseForCausalLM(config)
    model.save_pretrained(path, safe_serialization=True)
    PreTrainedTokenizerFast(tokenizer_object=tokenizer, eos_token="<eos>", pad_token="<pad>").save_pretrained(path)
    return model


def test_inference_tools_agree_on_one_device_and_split_over_two_ranks(tmp_path):
    """``lm_engine.cli.inference`` and ``lm_engine.cli.tensor_parallel_inference`` (two gloo ranks, each reading only its slices
    of the safetensors file) print the same continuations for a left-padded batch of prompts."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    model_path = str(tmp_path / "model")
    _tiny_model_with_tokenizer(model_path)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root)
    arguments = ["--model", model_path, "--prompt", "w3 w4 w5", "w9 w8", "--max-new-tokens", "6", "--dtype", "float32"]
    single = subprocess.run([sys.executable, "-m", "lm_engine.cli.inference", *arguments], env=env, capture_output=True, text=True,
                            cwd=str(tmp_path), timeout=600)
    assert single.returncode == 0, single.stderr[-2000:]
    split = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                            "--master-port", "29861", "-m", "lm_engine.cli.tensor_parallel_inference", *arguments], env=env,
                           capture_output=True, text=True, cwd=str(tmp_path), timeout=600)
    assert split.returncode == 0, split.stderr[-2000:]

    def continuations(text: str) -> list[str]:
        lines = text.splitlines()
        return [lines[i + 1] for i, line in enumerate(lines) if line.startswith("--- ")]

    assert len(continuations(single.stdout)) == 2 and all(len(line.split()) >= 1 for line in continuations(single.stdout))
    assert continuations(single.stdout) == continuations(split.stdout)


def test_conversion_tools_round_trip_and_pt_to_safetensors(tmp_path, capsys):
    """``import_from_hf`` -> ``export_to_hf`` gives back the Hugging Face weights; ``pt_to_safetensors`` turns a ``torch.save``
    checkpoint into safetensors that load to the same weights."""
    import os

    import torch
    from safetensors.torch import load_file
    from transformers import AutoConfig, AutoModelForCausalLM

    from lm_engine.cli import export_to_hf, import_from_hf, pt_to_safetensors

    torch.manual_seed(0)
    hf = AutoModelForCausalLM.from_config(AutoConfig.for_model(
        "llama", vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        max_position_embeddings=64, tie_word_embeddings=False)).float()
    hf_dir, ours_dir, back_dir = (str(tmp_path / name) for name in ("hf", "ours", "back"))
    hf.save_pretrained(hf_dir, safe_serialization=True)
    _run(import_from_hf, ["--model", hf_dir, "--save-path", ours_dir], capsys)
    _run(export_to_hf, ["--model", ours_dir, "--save-path", back_dir, "--model-type", "llama"], capsys)
    original = hf.state_dict()
    exported = {}
    for name in os.listdir(back_dir):
        if name.endswith(".safetensors"):
            exported.update(load_file(os.path.join(back_dir, name)))
    assert set(exported) == set(original) and all(torch.equal(exported[key], original[key]) for key in original)

    model = _tiny_model_with_tokenizer(str(tmp_path / "tiny"))
    pt_dir, st_dir = str(tmp_path / "pt"), str(tmp_path / "st")
    os.makedirs(pt_dir)
    model.config.save_pretrained(pt_dir)
    torch.save(model.state_dict(), os.path.join(pt_dir, "pytorch_model.bin"))
    _run(pt_to_safetensors, ["--model", pt_dir, "--save-path", st_dir, "--dtype", "float32"], capsys)
    saved = {}
    for name in os.listdir(st_dir):
        if name.endswith(".safetensors"):
            saved.update(load_file(os.path.join(st_dir, name)))
    for key, value in model.state_dict().items():
        assert torch.equal(saved[key], value), key


def test_whole_corpus_conversion_in_jobs_and_merge_by_size(tmp_path, capsys):
    """``convert-tree`` divides the files of every subset among jobs (together they convert each file once, a repeated job
    skips what is there); ``merge-tree`` joins the stores of a subset, in groups when a size limit is given, and records the
    grouping; the merged stores hold every document of the sources in order."""
    import os

    import pyarrow as pa

    from lm_engine.cli import preprocess_data
    from lm_engine.data.megatron.indexed_dataset import MMapIndexedDataset

    class Tokenizer:
        vocab_size, eos_token_id = 1000, 1

    raw, staged, merged = (str(tmp_path / name) for name in ("raw", "staged", "merged"))
    schema = pa.schema([pa.field("tokens", pa.uint32())])
    documents = {}
    for subset, files in (("a", 5), ("b", 2)):
        os.makedirs(os.path.join(raw, subset))
        for f in range(files):
            with pa.ipc.new_file(os.path.join(raw, subset, f"part{f}.arrow"), schema) as writer:
                for d in range(3):
                    tokens = [10 * f + d + 2] * (4 + d)
                    writer.write(pa.record_batch([pa.array(tokens, type=pa.uint32())], schema))
                    documents.setdefault(subset, []).append(tokens + [1])
    counts = [len(preprocess_data.convert_tree(Tokenizer(), raw, staged, ["a", "b"], jobs=3, job_index=job)) for job in range(3)]
    assert sum(counts) == 7 and max(counts) <= 4
    assert preprocess_data.convert_tree(Tokenizer(), raw, staged, ["a", "b"], jobs=1, job_index=0) == []  # all there already
    made = preprocess_data.merge_tree(staged, merged, ["a", "b"])
    assert sorted(made) == ["a", "b"] and len(made["a"]) == 5
    for subset in ("a", "b"):
        store = MMapIndexedDataset(os.path.join(merged, subset))
        assert [store[i].tolist() for i in range(len(store))] == documents[subset]
    grouped = preprocess_data.merge_tree(staged, str(tmp_path / "grouped"), ["a"], max_file_size=50 / 1024**3, output_suffix="v1")
    assert len(grouped) >= 2 and sum(len(group) for group in grouped.values()) == 5
    with open(tmp_path / "grouped" / "files-v1.json") as handle:
        assert json.load(handle) == grouped
    out = _run(preprocess_data, ["merge-tree", "--input-path", staged, "--output-path", str(tmp_path / "again"), "--data-subsets", "b"], capsys)
    assert "b: 2 stores" in out

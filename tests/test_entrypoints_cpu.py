"""The YAML-driven entry points run end to end on CPU: pretrain -> checkpoint -> unshard -> reload with
``from_pretrained`` -> generate; finetune on the synthetic debug dataset."""

import json
import os
import subprocess
import sys

import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(module: str, config: dict, tmp_path, name: str):
    path = tmp_path / f"{name}.yml"
    path.write_text(yaml.safe_dump(config))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29741")
    result = subprocess.run([sys.executable, "-m", module, "--config", str(path)], env=env, cwd=str(tmp_path), timeout=900,
                            capture_output=True, text=True)
    assert result.returncode == 0, result.stderr[-4000:]
    return result


def _tokenizer(tmp_path) -> str:
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from transformers import PreTrainedTokenizerFast

    vocab = {"<bos>": 0, "<eos>": 1, "<pad>": 2, "<unk>": 3}
    vocab.update({f"w{i}": i + 4 for i in range(60)})
    tok = Tokenizer(WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    path = tmp_path / "tokenizer"
    PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<bos>", eos_token="<eos>", pad_token="<pad>", unk_token="<unk>").save_pretrained(str(path))
    return str(path)


def _model_config(moe: bool = False) -> dict:
    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=64, add_bias=False)
    moe_block = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=32, add_bias=False, num_experts=4, num_experts_per_tok=2)
    return dict(model_type="gpt_base", vocab_size=64, hidden_size=32, num_layers=2, position_embedding_type="rope",
                normalization_function="rmsnorm", tie_word_embeddings=False, max_position_embeddings=64,
                bos_token_id=0, eos_token_id=1, pad_token_id=2,
                sequence_mixer_blocks=[attn, attn], mlp_blocks=[mlp, moe_block if moe else mlp])


def test_pretrain_unshard_generate(tmp_path):
    tokenizer = _tokenizer(tmp_path)
    save = tmp_path / "ckpt"
    pretrain = dict(
        datasets=[dict(class_name="SyntheticDataset", data_name="synthetic", class_args=dict(sequence_length=32, seed=3))],
        tokenizer_args=dict(tokenizer_name=tokenizer),
        model_args=dict(model_class="AutoModelForCausalLM", pretrained_config=_model_config(moe=True), use_padding_free_transformer=False),
        tuning_args=dict(tuning_method="pretraining"),
        save_args=dict(save_path=str(save), save_interval=4),
        training_parameters=dict(num_training_steps=4, micro_batch_size=2, gradient_accumulation_steps=2, eval_during_training=False),
        optimizer_args=dict(class_name="TorchAdamW", class_args=dict(lr=1e-3, weight_decay=0.1, betas=[0.9, 0.95], eps=1e-10)),
        lr_scheduler_args=dict(lr_decay_style="power", num_warmup_steps=1, extra_lr_scheduler_args=dict(a=0.5, b=-0.51, c=64)),
        mixed_precision_args=dict(dtype="fp32"),
        logging_args=dict(log_interval=2),
    )
    result = _run("lm_engine.pretrain", pretrain, tmp_path, "pretrain")
    assert "train-loss" in result.stderr or "train-loss" in result.stdout
    assert (save / "global_step4" / "model").is_dir()

    unsharded = tmp_path / "unsharded"
    _run("lm_engine.unshard", dict(load_args=dict(load_path=str(save)), unsharded_path=str(unsharded)), tmp_path, "unshard")
    assert (unsharded / "config.json").exists() and (unsharded / "model.safetensors").exists()

    sys.path.insert(0, ROOT)
    from lm_engine.hf_models import GPTBaseForCausalLM

    model = GPTBaseForCausalLM.from_pretrained(str(unsharded))
    ids = torch.randint(4, 64, (2, 8))
    out = model(input_ids=ids, labels=ids)
    assert torch.isfinite(out.loss)

    # generation from the unsharded model through the inference entry point (debug dataset = synthetic prompts)
    inference = dict(
        datasets=[dict(class_name="DebugDataset", data_name="debug", class_args=dict(num_examples=3), max_input_tokens=6, max_output_tokens=4)],
        model_args=dict(model_class="AutoModelForCausalLM", model_name=str(unsharded)),
        tokenizer_args=dict(tokenizer_name=tokenizer),
        generation_parameters=dict(batch_size=2, max_new_tokens=5, do_sample=False),
        output_dir=str(tmp_path / "generations"),
    )
    _run("lm_engine.generate", inference, tmp_path, "generate")
    lines = (tmp_path / "generations" / "output-debug.jsonl").read_text().strip().splitlines()
    assert len(lines) == 3 and "generated_text" in json.loads(lines[0])


def test_training_stops_before_saving_when_a_kernel_reported_a_timeout(tmp_path):
    """A status word raised by a kernel whose bounded wait ran out (made here on the host: the health check is replaced
    by one that reports status 4 at the first save point) ends the run before a checkpoint is written."""
    save = tmp_path / "ckpt"
    config = dict(
        datasets=[dict(class_name="SyntheticDataset", data_name="synthetic", class_args=dict(sequence_length=32, seed=3))],
        model_args=dict(model_class="AutoModelForCausalLM", pretrained_config=_model_config(), use_padding_free_transformer=False),
        tuning_args=dict(tuning_method="pretraining"),
        save_args=dict(save_path=str(save), save_interval=2),
        training_parameters=dict(num_training_steps=4, micro_batch_size=2, gradient_accumulation_steps=1, eval_during_training=False),
        optimizer_args=dict(class_name="TorchAdamW", class_args=dict(lr=1e-3)),
        lr_scheduler_args=dict(lr_decay_style="cosine", num_warmup_steps=1),
        mixed_precision_args=dict(dtype="fp32"),
        logging_args=dict(log_interval=100),
    )
    path = tmp_path / "pretrain.yml"
    path.write_text(yaml.safe_dump(config))
    driver = (
        "import lm_engine.pretrain as p\n"
        "def failing():\n"
        "    raise RuntimeError('a kernel on cuda:0 gave up waiting (status 4)')\n"
        "p.check_device_health = failing\n"
        f"p.main(argv=['--config', r'{path}'])\n"
    )
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29743")
    result = subprocess.run([sys.executable, "-c", driver], env=env, cwd=str(tmp_path), timeout=900, capture_output=True, text=True)
    assert result.returncode != 0
    assert "gave up waiting (status 4)" in result.stderr
    assert not (save / "latest_checkpointed_iteration.json").exists()
    assert not (save / "global_step2" / "model").exists()


def test_finetune_on_debug_dataset(tmp_path):
    tokenizer = _tokenizer(tmp_path)
    config = dict(
        datasets=[dict(class_name="DebugDataset", data_name="debug", class_args=dict(num_examples=32), data_sampling_ratio=1,
                       max_input_tokens=8, max_output_tokens=8)],
        tokenizer_args=dict(tokenizer_name=tokenizer),
        model_args=dict(model_class="AutoModelForCausalLM", pretrained_config=_model_config(), use_padding_free_transformer=True),
        tuning_args=dict(tuning_method="full_finetuning"),
        save_args=dict(save_path=str(tmp_path / "ft"), save_interval=3),
        training_parameters=dict(num_training_steps=3, micro_batch_size=4, gradient_accumulation_steps=2, eval_during_training=False),
        optimizer_args=dict(class_name="TorchAdamW", class_args=dict(lr=1e-3, weight_decay=0.0, betas=[0.9, 0.95], eps=1e-10)),
        lr_scheduler_args=dict(lr_decay_style="linear", num_warmup_steps=1),
        mixed_precision_args=dict(dtype="fp32"),
        logging_args=dict(log_interval=1),
    )
    result = _run("lm_engine.finetune", config, tmp_path, "finetune")
    assert (tmp_path / "ft" / "global_step3" / "dataloader" / "dataloader-0.pt").exists()
    text = result.stderr + result.stdout
    assert "train-loss" in text

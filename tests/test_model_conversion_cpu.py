"""HF import/export: logits of a random HF model equal the imported model's, and export(import(x)) == x."""

import os

import pytest
import torch
from transformers import AutoConfig, AutoModelForCausalLM

from lm_engine.hf_models import GPTBaseForCausalLM, export_to_huggingface, import_from_huggingface
from lm_engine.utils import SafeTensorsWeightsManager


def _hf_config(model_type: str):
    common = dict(vocab_size=96, hidden_size=32, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=64, tie_word_embeddings=False, bos_token_id=0, eos_token_id=1, pad_token_id=2)
    granite = dict(attention_multiplier=0.3, embedding_multiplier=1.7, residual_multiplier=0.6, logits_scaling=2.5)
    if model_type == "llama":
        return AutoConfig.for_model("llama", intermediate_size=48, **common)
    if model_type == "llama_bias":
        return AutoConfig.for_model("llama", intermediate_size=48, attention_bias=True, mlp_bias=True, **common)
    if model_type == "granite":
        return AutoConfig.for_model("granite", intermediate_size=48, **common, **granite)
    if model_type == "granitemoe":
        return AutoConfig.for_model("granitemoe", intermediate_size=24, num_local_experts=4, num_experts_per_tok=2, **common, **granite)
    if model_type == "granitemoeshared":
        return AutoConfig.for_model("granitemoeshared", intermediate_size=24, num_local_experts=4, num_experts_per_tok=2,
                                    shared_intermediate_size=40, **common, **granite)
    if model_type == "granitemoehybrid":
        return AutoConfig.for_model("granitemoehybrid", intermediate_size=24, num_local_experts=4, num_experts_per_tok=2,
                                    shared_intermediate_size=40, layer_types=["mamba", "attention", "mamba"], mamba_n_heads=4,
                                    mamba_d_state=8, mamba_n_groups=1, mamba_expand=2, mamba_d_conv=4, mamba_chunk_size=8,
                                    mamba_d_head=16, position_embedding_type="nope", **common, **granite)
    if model_type == "gpt_bigcode_mqa":
        return AutoConfig.for_model("gpt_bigcode", vocab_size=96, n_embd=32, n_layer=2, n_head=4, n_positions=64, multi_query=True,
                                    resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    if model_type == "gpt_bigcode_mha":
        return AutoConfig.for_model("gpt_bigcode", vocab_size=96, n_embd=32, n_layer=2, n_head=4, n_positions=64, multi_query=False,
                                    resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    raise ValueError(model_type)


@pytest.mark.parametrize("name", ["llama", "llama_bias", "granite", "granitemoe", "granitemoeshared", "granitemoehybrid",
                                  "gpt_bigcode_mqa", "gpt_bigcode_mha"])
def test_import_export_round_trip(name, tmp_path):
    torch.manual_seed(0)
    hf_config = _hf_config(name)
    hf_model = AutoModelForCausalLM.from_config(hf_config).eval().float()
    with torch.no_grad():  # non-trivial values everywhere (norm weights, biases)
        for p in hf_model.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    hf_dir, ours_dir, back_dir = (str(tmp_path / d) for d in ("hf", "ours", "back"))
    hf_model.save_pretrained(hf_dir, safe_serialization=True)

    import_from_huggingface(hf_dir, ours_dir)
    model = GPTBaseForCausalLM.from_pretrained(ours_dir).eval().float()

    ids = torch.randint(3, 96, (2, 24))
    with torch.no_grad():
        expected = hf_model(input_ids=ids).logits
        got = model(input_ids=ids).logits
    assert got.shape == expected.shape
    torch.testing.assert_close(got, expected, atol=2e-5, rtol=1e-4)

    export_to_huggingface(ours_dir, back_dir, hf_config.model_type)
    original, exported = SafeTensorsWeightsManager(hf_dir), SafeTensorsWeightsManager(back_dir)
    original_state = original.state_dict()
    exported_state = exported.state_dict()
    for key, value in original_state.items():
        if key == "lm_head.weight" and key not in exported_state:
            continue
        assert torch.equal(exported_state[key], value), key
    reloaded = AutoModelForCausalLM.from_pretrained(back_dir).eval().float()
    with torch.no_grad():
        torch.testing.assert_close(reloaded(input_ids=ids).logits, expected, atol=2e-5, rtol=1e-4)
    import json

    with open(os.path.join(back_dir, "config.json")) as handle:
        written = json.load(handle)
    assert written["architectures"] == [type(hf_model).__name__]  # serving stacks pick the model class by this key


_REFERENCE_CONVERTERS = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
import transformers
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm, export_to_huggingface, import_from_huggingface
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
# the reference reads `rope_theta` / `rope_scaling` off the transformers configs, which the installed transformers keeps under
# `rope_parameters`
for name in ("LlamaConfig", "GraniteConfig", "GraniteMoeConfig", "GraniteMoeSharedConfig"):
    cls = getattr(transformers, name)
    cls.rope_theta = property(lambda self: (self.__dict__.get("rope_parameters") or {}).get("rope_theta", 10000))
    cls.rope_scaling = property(lambda self: None)
for root, model_type in json.loads(sys.argv[2]).items():
    import_from_huggingface(root + "/hf", root + "/theirs")
    export_to_huggingface(root + "/theirs", root + "/theirs_back", model_type=model_type)
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "lm_engine")),
                    reason="reference is not installed under baseline/_ref")
def test_converted_checkpoints_equal_the_reference_s_converters(tmp_path):
    """llama (with and without biases), granite, granitemoe, granitemoeshared and granitemoehybrid: the directory this package's
    import writes holds the tensors and the config of the one the reference's import writes from the same Hugging Face
    checkpoint, and so does the export back (bit-equal tensors, equal ``config.json``). The reference's gpt_bigcode
    converter does not run against the installed transformers."""
    import json
    import subprocess
    import sys

    from safetensors.torch import load_file

    reference = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    jobs = {}
    for name in ("llama", "llama_bias", "granite", "granitemoe", "granitemoeshared", "granitemoehybrid"):
        root = str(tmp_path / name)
        torch.manual_seed(0)
        hf_config = _hf_config(name)
        AutoModelForCausalLM.from_config(hf_config).float().save_pretrained(root + "/hf", safe_serialization=True)
        import_from_huggingface(root + "/hf", root + "/mine")
        export_to_huggingface(root + "/mine", root + "/mine_back", hf_config.model_type)
        jobs[root] = hf_config.model_type
    done = subprocess.run([sys.executable, "-c", _REFERENCE_CONVERTERS, reference, json.dumps(jobs)], cwd=str(tmp_path),
                          env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), timeout=900, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]

    def tensors(folder: str) -> dict:
        out = {}
        for name in os.listdir(folder):
            if name.endswith(".safetensors"):
                out.update(load_file(os.path.join(folder, name)))
        return out

    def config(folder: str) -> dict:
        with open(os.path.join(folder, "config.json")) as handle:
            made = json.load(handle)
        made.pop("rope_parameters", None)  # rewritten by the child's patch of the reference's config class
        return made

    for root in jobs:
        for mine, theirs in ((root + "/mine", root + "/theirs"), (root + "/mine_back", root + "/theirs_back")):
            a, b = tensors(mine), tensors(theirs)
            assert set(a) == set(b), (mine, sorted(set(a) ^ set(b)))
            for key in a:
                assert a[key].shape == b[key].shape and torch.equal(a[key], b[key]), (mine, key)
            assert config(mine) == config(theirs), mine

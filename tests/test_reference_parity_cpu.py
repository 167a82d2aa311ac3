"""Checkpoint-format parity with the reference package (when it is installed under ``baseline/_ref``): a model of the
reference and a model of this package built from the same config exchange ``state_dict``s key for key and produce
the same loss; further down, everything else that can be compared with the reference on a CPU. The reference runs in a
child process because both packages are called ``lm_engine``."""

import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


# ----------------------------------------------------------------------------------------------------------------------
# The reference runs in ONE child process that stays up for the whole module: importing torch, transformers and the reference
# package costs far more than any of the comparisons. A request is a piece of source text and its arguments; the child runs it
# as a script would run (``sys.argv`` = ``["-c", <reference>, *arguments]``) and answers with the traceback, if any.
_SERVER = r"""
import json, os, sys, traceback
answers = os.fdopen(os.dup(1), "w")
os.dup2(2, 1)  # whatever the jobs print goes to the log, not into the answers
reference = sys.argv[1]
for line in sys.stdin:
    request = json.loads(line)
    sys.argv = ["-c", reference] + request["arguments"]
    try:
        exec(compile(request["code"], "<reference job>", "exec"), {"__name__": "__main__"})
        error = None
    except BaseException:
        error = traceback.format_exc()
    answers.write(json.dumps({"error": error}) + "\n")
    answers.flush()
"""
_server: dict = {}


def _stop_server() -> None:
    process = _server.pop("process", None)
    if process is not None:
        try:
            process.stdin.close()
            process.wait(timeout=30)
        except Exception:
            process.kill()


def _in_reference(code: str, *arguments: str, timeout: float = 900.0) -> None:
    """Runs ``code`` with ``arguments`` inside the child process that has the reference package on its path."""
    import atexit
    import json
    import select
    import tempfile

    if "process" not in _server:
        folder = tempfile.mkdtemp(prefix="reference_child_")
        _server["log"] = open(os.path.join(folder, "log.txt"), "w+")
        _server["process"] = subprocess.Popen([sys.executable, "-c", _SERVER, REF], cwd=folder, stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                              stderr=_server["log"], text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
        atexit.register(_stop_server)
    process = _server["process"]

    def log_tail() -> str:
        _server["log"].flush()
        _server["log"].seek(0)
        return _server["log"].read()[-3000:]

    process.stdin.write(json.dumps({"code": code, "arguments": [str(a) for a in arguments]}) + "\n")
    process.stdin.flush()
    ready, _, _ = select.select([process.stdout], [], [], timeout)
    if not ready:
        process.kill()
        _server.pop("process")
        raise AssertionError(f"the reference job did not finish within {timeout} s\n{log_tail()}")
    line = process.stdout.readline()
    if not line:
        _server.pop("process")
        raise AssertionError(f"the reference process ended (exit code {process.poll()})\n{log_tail()}")
    error = json.loads(line)["error"]
    assert error is None, error

_CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm, disable_generation_cache
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
blocks = [{"sequence_mixer_type": "softmax_attention", "num_attention_heads": 4, "num_key_value_heads": 2, "add_bias": False}] * 2
mlps = [{"mlp_type": "MLP", "activation_function": "swiglu", "intermediate_size": 128, "add_bias": False},
        {"mlp_type": "MoE", "activation_function": "swiglu", "intermediate_size": 64, "add_bias": False, "num_experts": 4, "num_experts_per_tok": 2}]
c = rm.GPTBaseConfig(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                     rope_theta=500000, sequence_mixer_blocks=blocks, mlp_blocks=mlps, tie_word_embeddings=False)
from transformers import AutoModelForCausalLM
torch.manual_seed(0)
m = AutoModelForCausalLM.from_config(c)
m.eval()
ids = torch.randint(0, 256, (2, 16))
with disable_generation_cache():
    out = m(input_ids=ids, labels=ids)
torch.save({"sd": m.state_dict(), "ids": ids, "loss": out.loss.detach(), "logits": out.logits.detach()}, sys.argv[2])
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_state_dict_and_loss_match_reference(tmp_path):
    out = tmp_path / "ref.pt"
    _in_reference(_CHILD, str(out))
    data = torch.load(out)

    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    blocks = [{"sequence_mixer_type": "softmax_attention", "num_attention_heads": 4, "num_key_value_heads": 2, "add_bias": False}] * 2
    mlps = [{"mlp_type": "MLP", "activation_function": "swiglu", "intermediate_size": 128, "add_bias": False},
            {"mlp_type": "MoE", "activation_function": "swiglu", "intermediate_size": 64, "add_bias": False, "num_experts": 4, "num_experts_per_tok": 2}]
    config = GPTBaseConfig(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           rope_theta=500000, sequence_mixer_blocks=blocks, mlp_blocks=mlps, tie_word_embeddings=False)
    model = GPTBaseForCausalLM(config)
    result = model.load_state_dict(data["sd"], strict=True)
    assert not result.missing_keys and not result.unexpected_keys
    model.eval()
    with torch.no_grad():
        mine = model(input_ids=data["ids"], labels=data["ids"])
    assert torch.allclose(mine.logits, data["logits"], atol=3e-6, rtol=1e-5)
    assert abs(mine.loss.item() - data["loss"].item()) < 1e-5


_COMMON = r"""
import sys, torch
import torch.distributed.checkpoint as dcp
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm, disable_generation_cache
from lm_engine.checkpointing.model import _ModelSaver
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
blocks = [{"sequence_mixer_type": "softmax_attention", "num_attention_heads": 4, "num_key_value_heads": 2, "add_bias": False}] * 2
mlps = [{"mlp_type": "MLP", "activation_function": "swiglu", "intermediate_size": 128, "add_bias": False},
        {"mlp_type": "MoE", "activation_function": "swiglu", "intermediate_size": 64, "add_bias": False, "num_experts": 4, "num_experts_per_tok": 2}]
c = rm.GPTBaseConfig(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                     rope_theta=500000, sequence_mixer_blocks=blocks, mlp_blocks=mlps, tie_word_embeddings=False)
from transformers import AutoModelForCausalLM
class Wrapper(torch.nn.Module):  # what the reference's savers see: a wrapper whose `.model` is the network
    def __init__(self, model):
        super().__init__()
        self.model = model
    def has_teacher_model(self):
        return False
torch.manual_seed(0)
wrapper = Wrapper(AutoModelForCausalLM.from_config(c))
wrapper.eval()
"""

_WRITE = _COMMON + r"""
ids = torch.randint(0, 256, (2, 16))
with disable_generation_cache():
    out = wrapper.model(input_ids=ids, labels=ids)
# the reference's own saver object through torch.distributed.checkpoint, as in its save_checkpoint (one process: no_dist)
dcp.save({"state": _ModelSaver([wrapper])}, checkpoint_id=sys.argv[2], no_dist=True)
torch.save({"ids": ids, "logits": out.logits.detach()}, sys.argv[3])
"""

_READ = _COMMON + r"""
for p in wrapper.parameters():
    torch.nn.init.zeros_(p)
dcp.load({"state": _ModelSaver([wrapper])}, checkpoint_id=sys.argv[2], no_dist=True)
data = torch.load(sys.argv[3])
with disable_generation_cache():
    out = wrapper.model(input_ids=data["ids"])
torch.save({"logits": out.logits.detach()}, sys.argv[4])
"""


def _our_wrapper():
    import torch.nn as nn

    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.parallel.engine import ShardedTrainingEngine

    blocks = [{"sequence_mixer_type": "softmax_attention", "num_attention_heads": 4, "num_key_value_heads": 2, "add_bias": False}] * 2
    mlps = [{"mlp_type": "MLP", "activation_function": "swiglu", "intermediate_size": 128, "add_bias": False},
            {"mlp_type": "MoE", "activation_function": "swiglu", "intermediate_size": 64, "add_bias": False, "num_experts": 4, "num_experts_per_tok": 2}]
    config = GPTBaseConfig(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           rope_theta=500000, sequence_mixer_blocks=blocks, mlp_blocks=mlps, tie_word_embeddings=False)

    class Wrapper(nn.Module):
        def __init__(self, model):
            super().__init__()
            self.model = model

    torch.manual_seed(11)
    wrapper = Wrapper(GPTBaseForCausalLM(config))
    wrapper._lm_engine = ShardedTrainingEngine(wrapper, compute_dtype=torch.float32, device=torch.device("cpu"))
    wrapper.eval()
    return wrapper


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_distributed_checkpoints_cross_load_with_the_reference(tmp_path):
    """Both directions through ``torch.distributed.checkpoint``: a ``model`` store written by the reference's own saver
    object loads into this package's engine-owned model (same logits as the reference computed), and a store written by
    this package's checkpoint code loads through the reference's saver object into the reference model (same logits as
    this package computed)."""
    import torch.distributed.checkpoint as dcp

    from lm_engine.checkpointing.core import _placeholders, get_model_state_dict, set_model_state_dict

    ref_store, ref_out = tmp_path / "ref_model", tmp_path / "ref_out.pt"
    _in_reference(_WRITE, str(ref_store), str(ref_out))
    data = torch.load(ref_out)

    wrapper = _our_wrapper()
    state = _placeholders(get_model_state_dict([wrapper]))
    dcp.load({"state": state}, checkpoint_id=str(ref_store), no_dist=True)
    set_model_state_dict([wrapper], state)
    wrapper._lm_engine.refresh_parameters()
    with torch.no_grad():
        mine = wrapper.model(input_ids=data["ids"])
    assert torch.allclose(mine.logits, data["logits"], atol=3e-6, rtol=1e-5)

    # the other way round, from fresh weights of this package
    wrapper = _our_wrapper()
    with torch.no_grad():
        logits = wrapper.model(input_ids=data["ids"]).logits
    our_store, back = tmp_path / "our_model", tmp_path / "back.pt"
    dcp.save({"state": get_model_state_dict([wrapper])}, checkpoint_id=str(our_store), no_dist=True)
    _in_reference(_READ, str(our_store), str(ref_out), str(back))
    assert torch.allclose(torch.load(back)["logits"], logits, atol=3e-6, rtol=1e-5)


_HYBRID = dict(
    initializer_range=0.1, layer_norm_epsilon=1e-5, hidden_size=512, num_layers=4, max_position_embeddings=512,
    normalization_function="rmsnorm", position_embedding_type="rope", rope_theta=10000, vocab_size=50304, tie_word_embeddings=False,
    m_width=9, m_emb=12, m_residual=0.22, init_method="mup", rope_dim=64,
    sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=16), dict(sequence_mixer_type="mamba2"),
                           dict(sequence_mixer_type="rnn"), dict(sequence_mixer_type="gru")],
    mlp_blocks=[dict(activation_function="swiglu", mlp_type="MLP"),
                dict(activation_function="swiglu", mlp_type="MoE", shared_intermediate_size=512),
                dict(activation_function="swiglu", mlp_type="MLP"), dict(activation_function="swiglu", mlp_type="MLP")])

_GROUPS = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm
from lm_engine.optimization.params_group import get_mup_group_with_names, get_normal_group_with_names
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
from transformers import AutoModelForCausalLM
with torch.device("meta"):
    network = AutoModelForCausalLM.from_config(rm.GPTBaseConfig(**json.loads(sys.argv[2])))
class Wrapper(torch.nn.Module):
    def __init__(self, model):
        super().__init__()
        self.model, self.config = model, model.config
    def has_teacher_model(self):
        return False
wrapper = Wrapper(network)
arguments = {"lr": 3e-4, "weight_decay": 0.1}
json.dump({"normal": get_normal_group_with_names(wrapper, arguments).get_param_names(),
           "mup": get_mup_group_with_names(wrapper, arguments).get_param_names()}, open(sys.argv[3], "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_parameter_groups_are_those_of_the_reference(tmp_path):
    """The hybrid model of the reference's own parameter-group test (attention, Mamba-2, RNN and GRU mixers, one MoE block with a
    shared expert, muP initialisation; reference tests/training/params_group/training_config.yml): the reference's grouping
    functions, run in a child process on its model, and this package's on its own model put the same parameter names, in
    the same order, into the same groups, for the plain and for the muP method."""
    import json

    from lm_engine.enums import ParamsGroupMethod
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.optimization.params_group import get_param_groups_with_names

    out = tmp_path / "groups.json"
    _in_reference(_GROUPS, json.dumps(_HYBRID), str(out))
    theirs = json.loads(out.read_text())
    with torch.device("meta"):
        model = GPTBaseForCausalLM(GPTBaseConfig(**_HYBRID))
    for key, method in (("normal", None), ("mup", ParamsGroupMethod.mup)):
        mine = {group: [f"model.{name}" for name in names] for group, names in get_param_groups_with_names(model, method).items()}
        assert mine == theirs[key], key
    assert len(theirs["mup"]["mup"]) == 24 and len(theirs["normal"]["no_weight_decay"]) == 32


def _family_cases() -> dict:
    attention = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mamba2 = dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=128, num_heads=8, conv_kernel_size=4, num_groups=2, chunk_size=8)
    latent = dict(sequence_mixer_type="multihead_latent_attention", num_attention_heads=4, query_compression_size=32,
                  key_value_compression_size=32, head_dim=16)
    convolution = dict(sequence_mixer_type="causal_convolution", in_channels=64, out_channels=64, kernel_size=3, num_groups=64,
                       activation_function="silu")
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=128, add_bias=False)

    def config(first_mixer, position="rope", **extra):
        made = dict(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type=position, normalization_function="rmsnorm",
                    max_position_embeddings=64, tie_word_embeddings=False, sequence_mixer_blocks=[first_mixer, dict(attention)],
                    mlp_blocks=[dict(mlp), dict(mlp)])
        if position == "rope":
            made["rope_dim"] = 16
        made.update(extra)
        return made

    biased_and_moe = [dict(mlp_type="MLP", activation_function="gelu_pytorch_tanh", intermediate_size=128, add_bias=True),
                      dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=64, shared_intermediate_size=32, num_experts=4,
                           num_experts_per_tok=2, add_bias=False)]
    # name -> (model family, config, tolerance of the logits); rnn / gru / stick-breaking are absent because the reference
    # cannot evaluate them without its kernel packages
    return {
        "mamba2": ("gpt_base", config(mamba2), 1e-4),
        "causal_convolution": ("gpt_base", config(convolution), 1e-6),
        "latent_attention_nope": ("gpt_base", config(latent, "nope"), 1e-6),
        "latent_attention_learned": ("gpt_base", config(latent, "learned_absolute"), 1e-6),
        "mup_multipliers": ("gpt_base", config(attention, m_emb=12, m_width=9, m_residual=0.22, init_method="mup"), 1e-6),
        "layernorm_bias_shared_expert": ("gpt_base", config(attention, "learned_absolute", normalization_function="layernorm",
                                                            mlp_blocks=biased_and_moe), 1e-6),
        "palm": ("palm", config(attention), 1e-6),
        "ladder_residual": ("ladder_residual", config(attention), 1e-6),
        "ladder_residual_mamba2": ("ladder_residual", config(mamba2), 1e-4),
        "gpt_crosslayer": ("gpt_crosslayer", config(attention), 1e-6),
        "gpt_crosslayer_shared": ("gpt_crosslayer", config(attention, sharing_pattern=[0, 0]), 1e-6),
    }


_FAMILIES = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm, disable_generation_cache
from transformers import AutoModelForCausalLM
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
classes = {"gpt_base": rm.GPTBaseConfig, "palm": rm.PaLMConfig, "ladder_residual": rm.LadderResidualConfig, "gpt_crosslayer": rm.GPTCrossLayerConfig}
for family in ("gpt_base", "palm", "ladder_residual"):  # classes without a constructor of their own
    classes[family].__init__ = init
import functools
cm.CommonConfig.__init__ = functools.wraps(orig)(init)  # reached through the constructor of the cross-layer config; keeps the signature
results = {}
for name, (family, config, _) in json.loads(sys.argv[2]).items():
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(classes[family](**config))
    model.eval()
    ids = torch.randint(0, config["vocab_size"], (2, 16))
    with disable_generation_cache(), torch.no_grad():
        out = model(input_ids=ids, labels=ids, use_cache=False)
    results[name] = {"sd": model.state_dict(), "ids": ids, "loss": out.loss, "logits": out.logits}
torch.save(results, sys.argv[3])
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_every_family_the_reference_can_evaluate_on_cpu_gives_its_logits(tmp_path):
    """Model families (gpt_base, palm, ladder_residual, gpt_crosslayer with and without shared keys / values) and mixers
    (Mamba-2, causal convolution, multi-head latent attention, muP multipliers, LayerNorm + biases + an MoE block with a
    shared expert): the reference's weights load key for key into this package's model of the same config, and the logits
    and the loss are the reference's (bit-equal but for Mamba-2, whose chunked scan sums in another order)."""
    import json

    import lm_engine.hf_models as hm

    cases = _family_cases()
    out = tmp_path / "families.pt"
    _in_reference(_FAMILIES, json.dumps(cases), str(out))
    theirs = torch.load(out)
    classes = {"gpt_base": (hm.GPTBaseConfig, hm.GPTBaseForCausalLM), "palm": (hm.PaLMConfig, hm.PaLMForCausalLM),
               "ladder_residual": (hm.LadderResidualConfig, hm.LadderResidualForCausalLM),
               "gpt_crosslayer": (hm.GPTCrossLayerConfig, hm.GPTCrossLayerForCausalLM)}
    for name, (family, config, tolerance) in cases.items():
        make_config, make_model = classes[family]
        model = make_model(make_config(**config))
        result = model.load_state_dict(theirs[name]["sd"], strict=True)
        assert not result.missing_keys and not result.unexpected_keys, name
        model.eval()
        with torch.no_grad():
            mine = model(input_ids=theirs[name]["ids"], labels=theirs[name]["ids"])
        assert (mine.logits - theirs[name]["logits"]).abs().max().item() <= tolerance, name
        assert abs(mine.loss.item() - theirs[name]["loss"].item()) <= 1e-5, name


_SCHEDULES = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
from lm_engine.enums import LRDecaySchedule
from lm_engine.optimization.scheduler import _LR_SCHEDULER_CLASSES
results = {}
for name, case in json.loads(sys.argv[2]).items():
    optimizer = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=case["lr"])
    scheduler = _LR_SCHEDULER_CLASSES[LRDecaySchedule(case["style"])](optimizer, **case["arguments"])
    results[name] = [scheduler._lr_lambda(step) for step in range(case["steps"])]
json.dump(results, open(sys.argv[3], "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_learning_rate_schedules_follow_the_reference_step_by_step(tmp_path):
    """Every decay style (constant, linear, cosine, exponential, power), with and without warm-up and constant phases, with an
    explicit decay length and with the one implied by the number of training steps, evaluated past its end: the factor of
    every step equals the one of the reference's scheduler classes (lm_engine/optimization/scheduler.py:56-196)."""
    import json

    from lm_engine.enums import LRDecaySchedule
    from lm_engine.optimization.scheduler import PhasedSchedule

    def arguments(warmup, constant, decay, total, floor, **extra):
        return dict(num_warmup_steps=warmup, num_constant_steps=constant, num_decay_steps=decay, num_training_steps=total,
                    lr_decay_factor=floor, **extra)

    cases = {}
    for style in ("linear", "cosine", "exponential"):
        cases[f"{style}_phases"] = dict(style=style, lr=3e-4, steps=80, arguments=arguments(5, 7, 40, 60, 0.1))
        cases[f"{style}_implied_length"] = dict(style=style, lr=3e-4, steps=80, arguments=arguments(0, 0, None, 60, 0.0))
    cases["constant"] = dict(style="constant", lr=1e-3, steps=30, arguments=arguments(4, 0, 0, 20, 0.1))
    cases["power"] = dict(style="power", lr=3e-4, steps=400, arguments=arguments(50, 0, None, 300, 0.1, a=4.6e-3, b=-0.51, c=16.0))
    cases["power_below_the_peak"] = dict(style="power", lr=0.02, steps=60, arguments=arguments(10, 0, None, 50, 0.1, a=0.03, b=-0.51, c=1.0))
    out = tmp_path / "schedules.json"
    _in_reference(_SCHEDULES, json.dumps(cases), str(out))
    theirs = json.loads(out.read_text())
    for name, case in cases.items():
        schedule = PhasedSchedule(LRDecaySchedule(case["style"]), base_lr=case["lr"], **case["arguments"])
        for step, expected in enumerate(theirs[name]):
            assert abs(schedule(step) - expected) <= 1e-12 * max(1.0, abs(expected)), (name, step, schedule(step), expected)


_TP_WEIGHTS = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm
from lm_engine.hf_models.models.gpt_base_TP.weights import (fix_gpt_base_unsharded_state_dict, get_gpt_base_model_parallel_state_dict,
                                                            unshard_gpt_base_tensor_parallel_state_dicts)
from lm_engine.utils import ProcessGroupManager, SafeTensorsWeightsManager
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
world = int(sys.argv[3])
for work, made in json.loads(sys.argv[2]).items():
    config = rm.GPTBaseConfig(**made)
    shards = []
    for rank in range(world):
        with ProcessGroupManager.set_dummy_tensor_parallel_world_size(world), ProcessGroupManager.set_dummy_tensor_parallel_rank(rank):
            shards.append(get_gpt_base_model_parallel_state_dict(config, SafeTensorsWeightsManager(work + "/model.safetensors"), 1, 0))
    mine = torch.load(work + "/shards.pt")
    with ProcessGroupManager.set_dummy_tensor_parallel_world_size(world):
        whole = unshard_gpt_base_tensor_parallel_state_dicts(config, mine["shards"])
        fixed = fix_gpt_base_unsharded_state_dict(config, dict(mine["concatenated"]), world)
    torch.save({"shards": shards, "whole": whole, "fixed": fixed}, work + "/theirs.pt")
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_tensor_parallel_weight_layout_is_the_reference_s(tmp_path):
    """Multi-query, grouped-query and multi-head attention with biases, a gated MLP with biases, a gated MoE block, learned
    positions and a vocabulary that needs padding, at tensor-parallel size 2: the per-rank state dicts cut by this package
    and by the reference (from the same safetensors file) are equal key for key and bit for bit; each side's unsharding of
    the other side's shards gives back the original weights; so does each side's repair of the rank-order concatenation
    (the form a tensor-parallel checkpoint is read back in)."""
    import json

    from safetensors.torch import save_file

    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.hf_models.tp_weights import _rule, fix_unsharded_state_dict, shard_state_dict, unshard_tensor_parallel_state_dicts

    world = 2
    cases = {}
    for key_value_heads in (1, 2, 4):
        attention = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=key_value_heads, add_bias=True)
        made = dict(vocab_size=250, hidden_size=64, num_layers=2, position_embedding_type="learned_absolute", max_position_embeddings=32,
                    normalization_function="layernorm", tie_word_embeddings=True, sequence_mixer_blocks=[attention, dict(attention)],
                    mlp_blocks=[dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=128, add_bias=True),
                                dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=64, num_experts=4, num_experts_per_tok=2,
                                     add_bias=False)])
        work = tmp_path / f"kv{key_value_heads}"
        work.mkdir()
        torch.manual_seed(3)
        model = GPTBaseForCausalLM(GPTBaseConfig(**made))
        config = model.config
        original = {k: v.detach().clone().contiguous() for k, v in model.state_dict().items() if k != "lm_head.weight"}
        save_file(original, str(work / "model.safetensors"))
        shards = [shard_state_dict(config, original, rank, world) for rank in range(world)]

        def dimension(key: str, config=config) -> int | None:  # along which a rank-order concatenation joins the pieces of a local tensor
            if ".kv_attn." in key:
                return None
            if ".q_attn." in key:
                return 0
            kind, dim, _ = _rule(config, key, world)
            return None if kind == "replicate" else dim

        concatenated = {key: shards[0][key] if dimension(key) is None else torch.cat([s[key] for s in shards], dim=dimension(key))
                        for key in shards[0]}
        torch.save({"shards": shards, "concatenated": concatenated}, work / "shards.pt")
        cases[str(work)] = (made, config, original, shards, concatenated)
    _in_reference(_TP_WEIGHTS, json.dumps({work: case[0] for work, case in cases.items()}), str(world))

    def same(a: dict, b: dict, skip=()) -> None:
        assert set(a) == set(b), (sorted(set(a) - set(b)), sorted(set(b) - set(a)))
        for key in a:
            if key not in skip:
                assert a[key].shape == b[key].shape and torch.equal(a[key], b[key]), key

    for work, (_, config, original, shards, concatenated) in cases.items():
        theirs = torch.load(os.path.join(work, "theirs.pt"))
        for rank in range(world):
            same(shards[rank], theirs["shards"][rank])
        same(theirs["whole"], original)
        same(unshard_tensor_parallel_state_dicts(config, theirs["shards"]), original)
        same(fix_unsharded_state_dict(config, concatenated, world), original)
        same(theirs["fixed"], original, skip=("transformer.wpe.weight",))  # the reference leaves the padding of the position table in


# the same scenario text runs against the reference (child process) and against this package (here): only the package that
# `lm_engine` resolves to differs
_DATA_SCENARIO = r"""
import torch
from lm_engine.data.base import BaseDataset, BlendedDatasets
from lm_engine.data.sampler import BlendedDistributedSampler
from lm_engine.data.utils import collate_fn
from lm_engine.enums import DatasetSplit, LossMask, Mode

class Tokenizer:
    eos_token_id = 2
    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": [3 + sum(map(ord, word)) % 97 for word in text.split()]}

class Words(BaseDataset):
    def __init__(self, name, count, mode, encoder_decoder=False, limits=(None, None), formats=("__input__", "__output__")):
        super().__init__(class_args={}, split=DatasetSplit.train, mode=mode, tokenizer=Tokenizer(), is_encoder_decoder=encoder_decoder,
                         data_name=name, input_format=formats[0], output_format=formats[1], max_input_tokens=limits[0],
                         max_output_tokens=limits[1])
        for i in range(count):
            prompt = self.construct_input_from_format(" ".join(f"{name}{i}w{j}" for j in range(1 + (i * 5) % 7)))
            answer = self.construct_output_from_format(" ".join(f"{name}{i}a{j}" for j in range(1 + (i * 3) % 5)))
            self.examples.append(self.get_input_output_token_ids(prompt, answer))

def scenario():
    results = {}
    # tokenisation: formats, trimming, end-of-sequence tokens, with and without outputs, decoder-only and encoder-decoder
    for label, kwargs in {
        "plain": dict(mode=Mode.training),
        "formatted": dict(mode=Mode.training, formats=("question: __input__ answer:", "__output__ .")),
        "trimmed": dict(mode=Mode.training, limits=(3, 3)),
        "inference": dict(mode=Mode.inference, limits=(4, None)),
        "encoder_decoder": dict(mode=Mode.training, encoder_decoder=True, limits=(4, 3)),
    }.items():
        results["examples_" + label] = Words("x", 9, **kwargs).examples
    # sampling order of a blend, per rank and epoch
    blend = BlendedDatasets([Words("a", 7, Mode.training), Words("b", 13, Mode.training), Words("c", 5, Mode.training)], DatasetSplit.train)
    results["blend_length"] = len(blend)
    results["blend_items"] = [blend[i] for i in (0, 6, 7, 19, 20, 24)]
    for shuffle in (False, True):
        for rank in range(4):
            sampler = BlendedDistributedSampler(blend, data_sampling_ratios=[3, 1, 2], num_replicas=4, rank=rank, shuffle=shuffle, seed=11)
            results[f"order_shuffle{int(shuffle)}_rank{rank}"] = [list(sampler), list(sampler)]
    sampler = BlendedDistributedSampler(blend, data_sampling_ratios=[1, 1, 1], num_replicas=2, rank=1, shuffle=True, seed=5, drop_last=True)
    results["order_drop_last"] = list(sampler)
    # collation
    batch = [dict(e) for e in Words("y", 5, Mode.training).examples]
    copy = lambda: [dict(input=list(e["input"]), output=list(e["output"])) for e in batch]
    def tensors(made):
        return {k: (v.tolist() if isinstance(v, torch.Tensor) else v) for k, v in made.items()}
    cpu = torch.device("cpu")
    results["collate_padded_output_only"] = tensors(collate_fn(copy(), Mode.training, LossMask.output_only, 2, False, False, pad_to_multiple_of=4, device=cpu))
    results["collate_packed_output_only"] = tensors(collate_fn(copy(), Mode.training, LossMask.output_only, 2, False, True, pad_to_multiple_of=8, device=cpu))
    results["collate_packed_no_mask"] = tensors(collate_fn(copy(), Mode.training, LossMask.no_mask, 2, False, True, device=cpu))
    results["collate_inference"] = tensors(collate_fn([dict(input=list(e["input"])) for e in batch], Mode.inference, LossMask.output_only, 2, False, False, device=cpu))
    # instruction-tuning corpora and SST-2 over a stand-in for `datasets.load_dataset`
    import datasets
    from lm_engine.data import AlpacaDataset, DollyDataset, SlimOrcaDataset, SST2Dataset
    corpora = {
        "tatsu-lab/alpaca": {"train": [dict(instruction="w1 w2", input="w3", output=" w4 w5 "), dict(instruction="w6", input="", output="w7")]},
        "databricks/databricks-dolly-15k": {"train": [dict(instruction="w1 w2", context="w3 w8", response="w4\n"), dict(instruction="w6", context="", response="w7")]},
        "Open-Orca/SlimOrca-Dedup": {"train": [dict(conversations=[dict(**{"from": "system"}, value="w9"), dict(**{"from": "human"}, value="w1 w2"), dict(**{"from": "gpt"}, value=" w4 ")]),
                                                dict(conversations=[dict(**{"from": "system"}, value=""), dict(**{"from": "human"}, value="w6"), dict(**{"from": "gpt"}, value="w7")])]},
        "sst2": {split: [dict(sentence=" w1 w2 ", label=1), dict(sentence="w3", label=0)] for split in ("train", "validation", "test")},
    }
    corpora["glue"] = corpora["sst2"]
    real, datasets.load_dataset = datasets.load_dataset, lambda name, *args, **kwargs: corpora[name]
    import sys
    for module in list(sys.modules.values()):  # modules that imported the function by name
        if getattr(module, "__name__", "").startswith("lm_engine.data") and hasattr(module, "load_dataset"):
            module.load_dataset = datasets.load_dataset
    try:
        for cls in (AlpacaDataset, DollyDataset, SlimOrcaDataset, SST2Dataset):
            for mode in (Mode.training, Mode.inference) if cls is SST2Dataset else (Mode.training,):
                made = cls(class_args={}, split=DatasetSplit.train, mode=mode, tokenizer=Tokenizer(), is_encoder_decoder=False, data_name="x",
                           input_format="__input__", output_format="__output__", max_input_tokens=None, max_output_tokens=None)
                results[f"{cls.__name__}_{mode.value}"] = made.examples
    finally:
        datasets.load_dataset = real
    from lm_engine.data import DebugDataset
    for label, class_args, mode in (("static", dict(num_examples=3, token_id=7), Mode.training), ("indexed", dict(num_examples=3, static_examples=False), Mode.training)):
        made = DebugDataset(class_args=class_args, split=DatasetSplit.train, mode=mode, tokenizer=Tokenizer(), is_encoder_decoder=False, data_name="d",
                            input_format="__input__", output_format="__output__", max_input_tokens=6, max_output_tokens=4)
        results["debug_" + label] = [len(made)] + [made[i] for i in range(len(made))]
    pairs = Words("z", 4, Mode.training, encoder_decoder=True).examples
    results["collate_encoder_decoder"] = tensors(collate_fn([dict(input=list(e["input"]), output=list(e["output"])) for e in pairs], Mode.training,
                                                            LossMask.output_only, 2, True, False, device=cpu))
    return results
"""

_DATA_CHILD = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
exec(sys.argv[2])
json.dump(scenario(), open(sys.argv[3], "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_finetuning_data_path_matches_the_reference(tmp_path):
    """Example construction (formats, trimming, end-of-sequence handling, inference and encoder-decoder forms), the order in
    which a blend of three datasets is sampled (with and without shuffling, four ranks, two epochs, drop_last) and the collated
    batches (padded, padding-free with padding of the token count, no-mask labels, inference, encoder-decoder) are those
    of the reference's classes, produced by the same scenario text run against either package."""
    import json

    out = tmp_path / "theirs.json"
    _in_reference(_DATA_CHILD, _DATA_SCENARIO, str(out))
    theirs = json.loads(out.read_text())
    scope: dict = {}
    exec(_DATA_SCENARIO, scope)
    mine = json.loads(json.dumps(scope["scenario"]()))
    assert set(mine) == set(theirs)
    for key in theirs:
        assert mine[key] == theirs[key], key


_TRAINING = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm
from transformers import AutoModelForCausalLM
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
config = json.loads(sys.argv[2])
torch.manual_seed(0)
model = AutoModelForCausalLM.from_config(rm.GPTBaseConfig(**config))
model.train()
ids = torch.randint(0, config["vocab_size"], (2, 16))
weights = {k: v.detach().clone() for k, v in model.state_dict().items()}
out = model(input_ids=ids, labels=ids, use_cache=False)
out.loss.backward()
torch.save({"sd": weights, "ids": ids, "loss": out.loss.detach(), "aux_loss": out.aux_loss.detach(),
            "grads": {n: p.grad for n, p in model.named_parameters()}}, sys.argv[3])
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_training_loss_with_router_loss_and_all_gradients_match_the_reference(tmp_path):
    """Training mode, an MoE block with a shared expert and a router auxiliary-loss coefficient: the total loss, the auxiliary
    loss and the gradient of every parameter equal the reference's from the same weights and tokens."""
    import json

    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    attention = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    made = dict(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                tie_word_embeddings=False, router_aux_loss_coef=0.02, sequence_mixer_blocks=[attention, dict(attention)],
                mlp_blocks=[dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=128, add_bias=False),
                            dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=64, shared_intermediate_size=32,
                                 num_experts=4, num_experts_per_tok=2, add_bias=False)])
    out = tmp_path / "training.pt"
    _in_reference(_TRAINING, json.dumps(made), str(out))
    theirs = torch.load(out)
    model = GPTBaseForCausalLM(GPTBaseConfig(**made))
    model.load_state_dict(theirs["sd"], strict=True)
    model.train()
    mine = model(input_ids=theirs["ids"], labels=theirs["ids"])
    assert abs(mine.loss.item() - theirs["loss"].item()) <= 1e-6
    assert abs(float(mine.aux_loss.detach()) - theirs["aux_loss"].item()) <= 1e-6
    mine.loss.backward()
    for name, parameter in model.named_parameters():
        expected = theirs["grads"][name]
        assert expected is not None and parameter.grad is not None, name
        assert (parameter.grad - expected).abs().max().item() <= 1e-5 * expected.abs().max().item() + 1e-9, name


_GREEDY = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm, disable_generation_cache
from transformers import AutoModelForCausalLM
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
results = {}
for name, case in json.loads(sys.argv[2]).items():
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(rm.GPTBaseConfig(**case["config"]))
    model.eval()
    ids = torch.randint(3, 256, (2, 7))
    mask = torch.ones_like(ids)
    mask[1, : case["padding"]] = 0
    sequence, attention, scores = ids, mask, []
    # the reference's own `generate` does not run against the installed transformers; greedy decoding by evaluating the whole
    # prefix again for every token needs its forward pass only
    with torch.no_grad(), disable_generation_cache():
        for _ in range(case["new_tokens"]):
            logits = model(input_ids=sequence, attention_mask=attention, use_cache=False).logits[:, -1]
            scores.append(logits)
            sequence = torch.cat([sequence, logits.argmax(-1, keepdim=True)], dim=1)
            attention = torch.cat([attention, torch.ones_like(attention[:, :1])], dim=1)
    results[name] = {"sd": model.state_dict(), "ids": ids, "mask": mask, "sequences": sequence, "scores": torch.stack(scores)}
torch.save(results, sys.argv[3])
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_cached_generation_repeats_the_reference_s_greedy_decoding(tmp_path):
    """``generate`` of this package (prefill + one token at a time from the KV / Mamba-2 caches) against greedy decoding
    with the reference's forward pass over the whole prefix: the same tokens and the same scores, for a left-padded batch
    through attention + MoE layers and for an unpadded batch through a Mamba-2 layer. (With left padding the reference's
    Mamba-2 block does not reproduce its own unpadded result, so that combination has nothing to compare with.)"""
    import json

    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    attention = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mamba2 = dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=128, num_heads=8, conv_kernel_size=4, num_groups=2, chunk_size=8)
    mlps = [dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=128, add_bias=False),
            dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=64, num_experts=4, num_experts_per_tok=2, add_bias=False)]

    def config(first):
        # end-of-sequence id outside the sampled range is not possible with 256 tokens: decoding is compared up to the first one
        return dict(vocab_size=256, hidden_size=64, num_layers=2, position_embedding_type="rope", rope_dim=16, normalization_function="rmsnorm",
                    tie_word_embeddings=False, bos_token_id=0, eos_token_id=1, pad_token_id=2, sequence_mixer_blocks=[first, dict(attention)],
                    mlp_blocks=mlps)

    cases = {"attention_left_padded": dict(config=config(attention), padding=3, new_tokens=9),
             "mamba2": dict(config=config(mamba2), padding=0, new_tokens=9)}
    out = tmp_path / "greedy.pt"
    _in_reference(_GREEDY, json.dumps(cases), str(out))
    theirs = torch.load(out)
    for name, case in cases.items():
        data = theirs[name]
        model = GPTBaseForCausalLM(GPTBaseConfig(**case["config"]))
        model.load_state_dict(data["sd"], strict=True)
        model.eval()
        made = model.generate(input_ids=data["ids"], attention_mask=data["mask"], max_new_tokens=case["new_tokens"], do_sample=False,
                              return_dict_in_generate=True, output_scores=True)
        prompt = data["ids"].shape[1]
        for row in range(data["ids"].shape[0]):
            expected = data["sequences"][row, prompt:].tolist()
            upto = expected.index(1) + 1 if 1 in expected else len(expected)  # this package stops a row at its end-of-sequence token
            assert made.sequences[row, prompt : prompt + upto].tolist() == expected[:upto], (name, row)
            for step in range(min(upto, len(made.scores))):
                assert (made.scores[step][row] - data["scores"][step][row]).abs().max().item() <= 1e-4, (name, row, step)


_SCHEMA = r"""
import enum, json, typing
import lm_engine.arguments as arguments
from pydantic import BaseModel

def fields_of(cls, seen):
    out = {}
    for name, field in cls.model_fields.items():
        nested = None
        for outer in [field.annotation, *typing.get_args(field.annotation)]:
            for inner in [outer, *typing.get_args(outer)]:
                if isinstance(inner, type) and issubclass(inner, BaseModel):
                    nested = inner
        default = field.default_factory() if field.default_factory is not None else field.default
        if isinstance(default, enum.Enum):
            default = default.value
        if isinstance(default, BaseModel):
            default = "<arguments>"
        try:
            json.dumps(default)
        except TypeError:
            default = repr(default)
        out[name] = {"default": default, "required": field.is_required()}
        if nested is not None and nested not in seen:
            out[name]["fields"] = fields_of(nested, seen | {nested})
    return out

def schema():
    return {name: fields_of(getattr(arguments, name), set())
            for name in ("TrainingArgs", "InferenceArgs", "UnshardingArgs", "DistillationArgs")}
"""

_SCHEMA_CHILD = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
exec(sys.argv[2])
json.dump(schema(), open(sys.argv[3], "w"))
"""

# keys this package adds to the reference's schema (all optional)
_ADDED_KEYS = {"fp8_recipe", "expert_parallel_world_size", "fused_collectives", "expert_capacity_factor", "keep_parameters_gathered", "strict"}


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_argument_schema_accepts_every_key_of_the_reference_with_its_default(tmp_path):
    """The four argument trees (training, inference, unsharding, distillation), walked recursively on both sides: every key
    of the reference exists here, is required or optional alike and has the same default, so a YAML file written for the
    reference means the same thing here; the only keys on top are the listed optional ones."""
    import json

    out = tmp_path / "schema.json"
    _in_reference(_SCHEMA_CHILD, _SCHEMA, str(out))
    theirs = json.loads(out.read_text())
    scope: dict = {}
    exec(_SCHEMA, scope)
    mine = json.loads(json.dumps(scope["schema"]()))
    problems, added = [], set()

    def compare(a: dict, b: dict, path: str) -> None:
        for key, entry in a.items():
            if key not in b:
                problems.append(f"missing: {path}{key}")
                continue
            if (entry["default"], entry["required"]) != (b[key]["default"], b[key]["required"]):
                problems.append(f"default of {path}{key}: {entry['default']!r} there, {b[key]['default']!r} here")
            if "fields" in entry:
                if "fields" not in b[key]:
                    problems.append(f"not a group here: {path}{key}")
                else:
                    compare(entry["fields"], b[key]["fields"], f"{path}{key}.")
        added.update(key for key in b if key not in a)

    for name in theirs:
        compare(theirs[name], mine[name], name + ".")
    assert not problems, problems
    assert added <= _ADDED_KEYS, added - _ADDED_KEYS


_MODEL_SCHEMA = r"""
import importlib, inspect
import lm_engine.hf_models.config as base

def model_schema():
    try:  # the reference keeps the block arguments in submodules of a package
        modules = [importlib.import_module("lm_engine.hf_models.config.mlp"), importlib.import_module("lm_engine.hf_models.config.sequence_mixer")]
    except ImportError:
        modules = [base]
    out = {}
    for module in modules:
        for name, cls in vars(module).items():
            if name.startswith("_") and hasattr(cls, "model_fields"):
                out[name] = {key: "<required>" if field.is_required() else repr(field.default_factory() if field.default_factory else field.default)
                             for key, field in cls.model_fields.items()}
    signature = inspect.signature(base.CommonConfig.__init__)
    out["CommonConfig"] = {key: repr(parameter.default) for key, parameter in signature.parameters.items() if key not in ("self", "kwargs")}
    return out
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_model_config_takes_the_reference_s_keys_and_defaults(tmp_path):
    """Constructor arguments of the common model config and the argument classes of every sequence-mixer and MLP block type:
    the same names with the same defaults on both sides."""
    import json

    out = tmp_path / "model_schema.json"
    child = "import json, sys\nsys.path.insert(0, sys.argv[1])\nexec(sys.argv[2])\njson.dump(model_schema(), open(sys.argv[3], 'w'))\n"
    _in_reference(child, _MODEL_SCHEMA, str(out))
    theirs = json.loads(out.read_text())
    scope: dict = {}
    exec(_MODEL_SCHEMA, scope)
    mine = scope["model_schema"]()
    assert len(theirs) == 10 and len(theirs["CommonConfig"]) > 20  # nine block argument classes and the config itself
    for name, fields in theirs.items():
        assert name in mine, name
        assert mine[name] == fields, (name, {k: (v, mine[name].get(k)) for k, v in fields.items() if mine[name].get(k) != v})


_PUBLIC_NAMES = r"""
import importlib, json, sys
sys.path.insert(0, sys.argv[1])
modules = json.loads(sys.argv[2])
found = {}
for name in modules:
    module = importlib.import_module(name)
    # what the module (or, for a package, one of its submodules) defines itself: names it merely imports from elsewhere are not its interface
    found[name] = sorted(key for key, value in vars(module).items() if not key.startswith("_") and not isinstance(value, type(sys))
                         and str(getattr(value, "__module__", "")).startswith(name))
import enum
import lm_engine.enums as enums
from lm_engine.optimization.optimizer import _OPTIMIZER_CLASSES
found["<enums>"] = {name: {member.name: member.value for member in cls} for name, cls in vars(enums).items()
                    if isinstance(cls, type) and issubclass(cls, enum.Enum) and cls is not enum.Enum}
found["<optimizers>"] = sorted(_OPTIMIZER_CLASSES)
json.dump(found, open(sys.argv[3], "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_public_names_of_the_reference_resolve_here(tmp_path):
    """Every public class and function that a package or entry-point module of the reference defines and exposes at its top
    level (``from lm_engine.hf_models import ...``, ``from lm_engine.data import ...`` and so on) can be imported from the module
    of the same name here."""
    import importlib
    import json

    modules = ["lm_engine.hf_models", "lm_engine.utils", "lm_engine.enums", "lm_engine.data", "lm_engine.data.megatron", "lm_engine.optimization",
               "lm_engine.checkpointing", "lm_engine.model_wrapper", "lm_engine.containers", "lm_engine.kernels", "lm_engine.distributed",
               "lm_engine.train_utils", "lm_engine.arguments", "lm_engine.communication", "lm_engine.dtensors", "lm_engine.gradient_checkpointing",
               "lm_engine.fp8", "lm_engine.defaults", "lm_engine.hf_models.model_conversion", "lm_engine.pretrain", "lm_engine.finetune",
               "lm_engine.generate", "lm_engine.unshard", "lm_engine.distill"]
    out = tmp_path / "names.json"
    _in_reference(_PUBLIC_NAMES, json.dumps(modules), str(out))
    theirs = json.loads(out.read_text())
    # every member of every enum (kernel names, modes, schedules, ...) with its value, and every optimizer name of the YAML files
    import lm_engine.enums as enums
    from lm_engine.optimization.optimizer import build_optimizer  # noqa: F401  (the module defines the table below)
    import lm_engine.optimization.optimizer as optimizer_module

    their_enums, their_optimizers = theirs.pop("<enums>"), theirs.pop("<optimizers>")
    assert len(their_enums) >= 10
    for name, members in their_enums.items():
        mine = {member.name: member.value for member in getattr(enums, name)}
        assert all(mine.get(key) == value for key, value in members.items()), (name, members, mine)
    known = {key for table in vars(optimizer_module).values() if isinstance(table, dict) for key in table if isinstance(key, str)}
    assert set(their_optimizers) <= known, set(their_optimizers) - known
    assert sum(len(names) for names in theirs.values()) > 150
    # helpers of the reference's own wrapping of torch FSDP / its data broadcast that have no counterpart in this design
    internal = {"lm_engine.data.megatron": {"get_source_and_broadcast_group"}, "lm_engine.kernels": {"is_cute_kernels_available"}}
    missing = {}
    for name, names in theirs.items():
        module = importlib.import_module(name)
        gone = [key for key in names if not hasattr(module, key) and key not in internal.get(name, ())]
        if gone:
            missing[name] = gone
    assert not missing, missing


_MEMBERS = r"""
import importlib, inspect, json, sys
sys.path.insert(0, sys.argv[1])
found = {}
for module_name, classes in json.loads(sys.argv[2]).items():
    module = importlib.import_module(module_name)
    for class_name in classes:
        cls = getattr(module, class_name)
        names = []
        for name, _ in inspect.getmembers(cls):
            if name.startswith("_"):
                continue
            owner = next((base for base in cls.__mro__ if name in vars(base)), None)
            if owner is not None and owner.__module__.startswith("lm_engine"):  # not what torch / transformers / pydantic bring along
                names.append(name)
        found[class_name] = names
json.dump(found, open(sys.argv[3], "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_public_methods_of_the_reference_s_main_classes_exist_here(tmp_path):
    """Process-group manager (every getter and every ``set_dummy_*`` context manager), communication helpers, step tracker,
    experiment tracker, metrics dict, safetensors manager, containers, model wrappers, generation cache, datasets, sampler and
    data loaders: every public method or attribute that the reference's class defines is there under the same name."""
    import importlib
    import json

    classes = {"lm_engine.utils": ["ProcessGroupManager", "StepTracker", "ExperimentsTracker", "MetricsTrackingDict", "SafeTensorsWeightsManager",
                                   "ProgressBar", "BaseArgs"],
               "lm_engine.communication": ["Communication"],
               "lm_engine.containers": ["ModelContainer", "OptimizerContainer", "LRSchedulerContainer", "BackwardHookOptimizerContainer"],
               "lm_engine.model_wrapper": ["ModelWrapper", "ModelWrapperForPretraining", "ModelWrapperForFinetuning", "ModelWrapperForDistillation"],
               "lm_engine.hf_models": ["GPTBaseForCausalLM", "GPTBaseModel"], "lm_engine.hf_models.cache": ["GenerationCache"],
               "lm_engine.data": ["ResumableDataLoader", "DispatchingDataLoader", "BlendedDatasets", "BaseDataset", "BlendedDistributedSampler"]}
    out = tmp_path / "members.json"
    _in_reference(_MEMBERS, json.dumps(classes), str(out))
    theirs = json.loads(out.read_text())
    assert len(theirs["ProcessGroupManager"]) > 25
    # set-up steps of the reference's wrappers / model that happen inside the constructors here
    internal = {"ModelWrapperForPretraining": {"reset_parameters"}, "ModelWrapperForDistillation": {"reset_parameters"}, "GPTBaseModel": {"mask_value"}}
    missing = {}
    for module_name, names in classes.items():
        module = importlib.import_module(module_name)
        for class_name in names:
            cls = getattr(module, class_name)
            gone = [name for name in theirs[class_name] if not hasattr(cls, name) and name not in internal.get(class_name, ())]
            if gone:
                missing[class_name] = gone
    assert not missing, missing


_CONFIG_FILES = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm
from transformers import AutoConfig
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
rm.GPTBaseConfig(**json.loads(sys.argv[2])).save_pretrained(sys.argv[3] + "/theirs")
views = {}
for which in ("theirs", "mine"):
    view = AutoConfig.from_pretrained(sys.argv[3] + "/" + which).to_dict()
    view.pop("_name_or_path", None)
    views[which] = json.loads(json.dumps(view, default=repr))
json.dump(views, open(sys.argv[3] + "/views.json", "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_config_files_are_interchangeable_with_the_reference(tmp_path):
    """A hybrid config (attention with a multiplier, Mamba-2, GRU, MoE with a shared expert, muP multipliers, YaRN scaling):
    ``config.json`` written by this package has the keys and values of the one the reference writes, the reference reads
    both into the same config, and this package reads the reference's file into the config it started from."""
    import json

    from transformers import AutoConfig

    from lm_engine.hf_models import GPTBaseConfig

    made = dict(vocab_size=256, hidden_size=64, num_layers=3, position_embedding_type="rope", rope_dim=16, normalization_function="rmsnorm",
                tie_word_embeddings=False, m_emb=12.0, m_width=2.0, m_residual=0.3, init_method="mup", router_aux_loss_coef=0.02,
                rope_scaling=dict(type="yarn", factor=4.0, original_max_position_embeddings=128),
                sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False,
                                            attention_multiplier=0.3),
                                       dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=128, num_heads=8, num_groups=2, chunk_size=8),
                                       dict(sequence_mixer_type="gru", state_size=32, num_heads=4)],
                mlp_blocks=[dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=128, add_bias=False),
                            dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=64, shared_intermediate_size=32, num_experts=4,
                                 num_experts_per_tok=2, add_bias=False),
                            dict(mlp_type="MLP", activation_function="gelu_pytorch_tanh", add_bias=True)])
    config = GPTBaseConfig(**made)
    config.save_pretrained(str(tmp_path / "mine"))
    _in_reference(_CONFIG_FILES, json.dumps(made), str(tmp_path))
    mine = json.loads((tmp_path / "mine" / "config.json").read_text())
    theirs = json.loads((tmp_path / "theirs" / "config.json").read_text())
    assert mine == theirs, {key: (mine.get(key), theirs.get(key)) for key in set(mine) | set(theirs) if mine.get(key) != theirs.get(key)}
    views = json.loads((tmp_path / "views.json").read_text())
    assert views["mine"] == views["theirs"]
    read_back = AutoConfig.from_pretrained(str(tmp_path / "theirs")).to_dict()
    expected = config.to_dict()
    for view in (read_back, expected):
        view.pop("_name_or_path", None)
    assert read_back == expected


_FLOPS_SCENARIO = r"""
import lm_engine.hf_models as hm
from lm_engine.enums import GradientCheckpointingMethod
from lm_engine.train_utils import get_model_tflops

def scenario():
    attention = dict(sequence_mixer_type="softmax_attention", num_attention_heads=8, num_key_value_heads=2, add_bias=False)
    mqa = dict(sequence_mixer_type="softmax_attention", num_attention_heads=8, num_key_value_heads=1, add_bias=True)
    mamba = dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=256, num_heads=8, num_groups=2, chunk_size=8)
    gru = dict(sequence_mixer_type="gru", state_size=64, num_heads=4)
    rnn = dict(sequence_mixer_type="rnn", state_size=64, num_heads=4)
    latent = dict(sequence_mixer_type="multihead_latent_attention", num_attention_heads=8, query_compression_size=64, key_value_compression_size=32, head_dim=16)
    conv = dict(sequence_mixer_type="causal_convolution", in_channels=128, out_channels=128, kernel_size=3, num_groups=128, activation_function="silu")
    sb = dict(sequence_mixer_type="stickbreaking_attention", num_attention_heads=8, num_key_value_heads=2)
    dense = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=512, add_bias=False)
    plain = dict(mlp_type="MLP", activation_function="gelu_pytorch_tanh", intermediate_size=512, add_bias=True)
    moe = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=128, num_experts=8, num_experts_per_tok=2, add_bias=False)
    shared = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=128, shared_intermediate_size=64, num_experts=8, num_experts_per_tok=2, add_bias=False)
    out = {}
    for name, mixers, mlps, extra in [
        ("dense", [attention] * 2, [dense] * 2, {}),
        ("mqa_plain", [mqa] * 2, [plain] * 2, dict(position_embedding_type="learned_absolute")),
        ("moe", [attention] * 2, [moe, shared], {}),
        ("hybrid", [mamba, gru, rnn, attention], [dense, moe, plain, dense], dict(num_layers=4)),
        ("latent_conv", [latent, conv], [dense] * 2, dict(position_embedding_type="nope")),
        ("stickbreaking", [sb] * 2, [dense] * 2, dict(position_embedding_type="nope")),
        ("tied", [attention] * 2, [dense] * 2, dict(tie_word_embeddings=True)),
    ]:
        made = dict(vocab_size=1000, hidden_size=128, num_layers=2, position_embedding_type="rope", rope_dim=16, normalization_function="rmsnorm",
                    tie_word_embeddings=False, sequence_mixer_blocks=[dict(m) for m in mixers], mlp_blocks=[dict(m) for m in mlps])
        made.update(extra)
        try:
            config = hm.GPTBaseConfig(**made)
            out[name] = [get_model_tflops(config, 16, 512, None, {}),
                         get_model_tflops(config, 4, 2048, GradientCheckpointingMethod.block, {}),
                         get_model_tflops(config, 4, 2048, GradientCheckpointingMethod.block, {"num_blocks": 1})]
        except Exception as error:
            out[name] = f"{type(error).__name__}: {error}"
    return out
"""

_FLOPS_CHILD = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
exec(sys.argv[2])
json.dump(scenario(), open(sys.argv[3], "w"))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_model_flop_count_is_the_reference_s(tmp_path):
    """The FLOP model behind the logged TFLOP/s and MFU (lm_engine/train_utils.py:73-212): dense, multi-query with biases, MoE
    with and without a shared expert, a Mamba-2 / GRU / RNN / attention hybrid, latent attention with a convolution mixer,
    stick-breaking attention and tied embeddings, each without recomputation, with every block recomputed and with one block
    recomputed, give the reference's numbers exactly."""
    import json

    out = tmp_path / "flops.json"
    _in_reference(_FLOPS_CHILD, _FLOPS_SCENARIO, str(out))
    theirs = json.loads(out.read_text())
    scope: dict = {}
    exec(_FLOPS_SCENARIO, scope)
    mine = json.loads(json.dumps(scope["scenario"]()))
    assert len(theirs) == 7 and all(isinstance(values, list) and min(values) > 0 for values in theirs.values()), theirs
    assert mine == theirs


_INITIAL_WEIGHTS = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
import lm_engine.hf_models as rm
from lm_engine.hf_models import config as cm
from transformers import AutoModelForCausalLM
orig = cm.CommonConfig.__init__
def init(self, *a, **k):
    orig(self, *a, **k)
    rope = self.__dict__.get("rope_parameters")
    if isinstance(rope, dict) and "factor" not in rope:
        self.__dict__["rope_parameters"] = None
rm.GPTBaseConfig.__init__ = init
made = {}
for name, config in json.loads(sys.argv[2]).items():
    torch.manual_seed(1234)
    made[name] = dict(AutoModelForCausalLM.from_config(rm.GPTBaseConfig(**config)).state_dict())
torch.save(made, sys.argv[3])
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_the_same_seed_gives_the_reference_s_initial_weights(tmp_path):
    """Initialisation (standard deviations by parameter kind, depth scaling of the output projections, muP division by the
    width multiplier, Mamba-2's ``A_log`` / ``dt_bias`` / ``D``, biases and norms) and the order in which the parameters draw
    from the generator: a model built here after ``torch.manual_seed(s)`` starts from exactly the weights of the
    reference's model built after the same call, for plain and for muP initialisation."""
    import json

    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    base = dict(
        vocab_size=512, hidden_size=256, num_layers=3, position_embedding_type="learned_absolute", max_position_embeddings=128,
        normalization_function="layernorm", tie_word_embeddings=False, initializer_range=0.02,
        sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=8, num_key_value_heads=2, add_bias=True),
                               dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=512, num_heads=8, num_groups=2, chunk_size=8),
                               dict(sequence_mixer_type="multihead_latent_attention", num_attention_heads=8, query_compression_size=64,
                                    key_value_compression_size=64, head_dim=32)],
        mlp_blocks=[dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=512, add_bias=True),
                    dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=256, shared_intermediate_size=128, num_experts=4,
                         num_experts_per_tok=2, add_bias=False),
                    dict(mlp_type="MLP", activation_function="gelu_pytorch_tanh", intermediate_size=512, add_bias=False)])
    cases = {"normal": base, "mup": dict(base, init_method="mup", m_width=4.0, m_emb=2.0, m_residual=0.5)}
    out = tmp_path / "initial.pt"
    _in_reference(_INITIAL_WEIGHTS, json.dumps(cases), str(out))
    theirs = torch.load(out)
    for name, config in cases.items():
        torch.manual_seed(1234)
        mine = GPTBaseForCausalLM(GPTBaseConfig(**config)).state_dict()
        assert set(mine) == set(theirs[name]) and len(mine) > 50
        for key, value in theirs[name].items():
            assert torch.equal(mine[key], value), (name, key)

"""Training-side pieces that need no GPU: blended sampling over simulated ranks, resumable / dispatching loaders,
JSON-lines datasets, optimizer parameter groups and the metrics accumulator
(the counterparts of tests/training/{blended_datasets,dataloader,jsonlines}_test.py and params_group/ of the reference)."""

import json

import pytest
import torch

from lm_engine.enums import DatasetSplit, Mode, ParamsGroupMethod


class _Tokenizer:
    eos_token_id = 1

    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": [2 + (ord(c) % 50) for c in text]}


def _debug_datasets(sizes, split=DatasetSplit.train):
    from lm_engine.data.base import BlendedDatasets
    from lm_engine.data.debug import DebugDataset
    from lm_engine.defaults import INPUT_FORMAT, OUTPUT_FORMAT

    datasets = [
        DebugDataset(class_args={"num_examples": n, "token_id": 5 + i}, split=split, mode=Mode.training, tokenizer=_Tokenizer(),
                     is_encoder_decoder=False, data_name=f"debug{i}", input_format=INPUT_FORMAT, output_format=OUTPUT_FORMAT,
                     max_input_tokens=4, max_output_tokens=4)
        for i, n in enumerate(sizes)
    ]
    return BlendedDatasets(datasets, split)


def test_blended_datasets_index_every_example_once():
    blended = _debug_datasets([100, 200, 300])
    assert len(blended) == 600 and blended.get_num_datasets() == 3
    assert blended.get_num_examples_in_each_dataset() == [100, 200, 300]
    first_token = [blended[i]["input"][0] for i in (0, 99, 100, 299, 300, 599)]
    assert first_token == [5, 5, 6, 6, 7, 7]


@pytest.mark.parametrize("shuffle", [False, True])
def test_blended_sampler_partitions_the_epoch_over_eight_ranks(shuffle):
    """Eight simulated ranks draw disjoint slices whose union is the epoch; per-dataset counts follow the ratios."""
    from lm_engine.data.sampler import BlendedDistributedSampler

    blended = _debug_datasets([100, 200, 300])
    world = 8
    per_rank = []
    for rank in range(world):
        sampler = BlendedDistributedSampler(blended, data_sampling_ratios=[1, 1, 2], num_replicas=world, rank=rank, shuffle=shuffle, seed=7)
        per_rank.append(list(sampler))
    assert len({len(x) for x in per_rank}) == 1
    everything = [i for x in per_rank for i in x]
    assert len(everything) == world * len(per_rank[0]) == 600
    by_dataset = [0, 0, 0]
    for i in everything:
        by_dataset[0 if i < 100 else (1 if i < 300 else 2)] += 1
    assert by_dataset == [150, 150, 300]  # ratios 1 : 1 : 2 of the 600 draws
    if not shuffle:
        assert per_rank[0][:3] == [0, 8, 16]  # rank-strided deal of the unshuffled index list


def test_blended_sampler_resumes_in_the_middle_of_an_epoch():
    from lm_engine.data.sampler import BlendedDistributedSampler

    blended = _debug_datasets([50, 70])
    make = lambda: BlendedDistributedSampler(blended, data_sampling_ratios=[1, 1], num_replicas=2, rank=1, shuffle=True, seed=3)
    reference = list(make())
    first = make()
    iterator = iter(first)
    head = [next(iterator) for _ in range(17)]
    state = first.state_dict()
    second = make()
    second.load_state_dict(state)
    # the resumed sampler continues the interrupted epoch where the first one stopped
    assert head == reference[:17]
    tail = []
    for i in second:
        tail.append(i)
    assert second.index == len(reference)


def test_resumable_dataloader_round_trips_its_state():
    from lm_engine.data.dataloader import ResumableDataLoader
    from lm_engine.data.sampler import BlendedDistributedSampler

    blended = _debug_datasets([40, 24])
    collate = lambda batch: [example["input"][0] for example in batch]

    def make():
        sampler = BlendedDistributedSampler(blended, data_sampling_ratios=[1, 1], num_replicas=1, rank=0, shuffle=True, seed=11)
        return ResumableDataLoader(blended, batch_size=4, sampler=sampler, collate_fn=collate, drop_last=True)

    full = [batch for batch in make()]
    loader = make()
    iterator = iter(loader)
    seen = [next(iterator) for _ in range(5)]
    state = loader.state_dict()
    assert seen == full[:5] and set(state) >= {"sampler"}
    resumed = make()
    resumed.load_state_dict(state)
    assert resumed.sampler.index == loader.sampler.index


@pytest.mark.parametrize("split", [DatasetSplit.train, DatasetSplit.val, DatasetSplit.test])
def test_jsonlines_directory_loads_every_file_of_the_split(tmp_path, split):
    """A directory with train / validation / test sub-directories of .jsonl files, read through the datasets library."""
    pytest.importorskip("datasets")
    from lm_engine.data.huggingface import HuggingFaceDataset
    from lm_engine.defaults import INPUT_FORMAT, OUTPUT_FORMAT

    name = {"train": "train", "val": "validation", "test": "test"}[split.value]
    folder = tmp_path / name
    folder.mkdir()
    for i in range(3):
        with open(folder / f"part{i}.jsonl", "w") as handle:
            for j in range(5):
                handle.write(json.dumps({"input": f"question {i} {j}", "output": f"answer {j}"}) + "\n")
    dataset = HuggingFaceDataset(class_args={"data_path": str(tmp_path)}, split=split, mode=Mode.training, tokenizer=_Tokenizer(),
                                 is_encoder_decoder=False, data_name="jsonl", input_format=INPUT_FORMAT, output_format=OUTPUT_FORMAT,
                                 max_input_tokens=64, max_output_tokens=64)
    assert len(dataset) == 15
    example = dataset[0]
    assert example["input"][-len(example["output"]):] == example["output"] and example["output"][-1] == _Tokenizer.eos_token_id


def _tiny_model(init_method="normal", m_width=None):
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    config = GPTBaseConfig(
        vocab_size=64, hidden_size=32, num_layers=2, max_position_embeddings=32, position_embedding_type="learned_absolute",
        normalization_function="layernorm", init_method=init_method, m_width=m_width,
        sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=True),
                               dict(sequence_mixer_type="rnn", state_size=32, num_heads=4, add_bias=True)],
        mlp_blocks=[dict(mlp_type="MLP", activation_function="gelu_pytorch_tanh", intermediate_size=64, add_bias=True),
                    dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=32, num_experts=4, num_experts_per_tok=2, add_bias=False)],
    )
    return GPTBaseForCausalLM(config)


def test_parameter_groups_split_decay_from_no_decay():
    from lm_engine.optimization.params_group import get_param_groups_with_names, get_torch_param_groups

    model = _tiny_model()
    groups = get_param_groups_with_names(model, None)
    assert set(groups) == {"normal", "no_weight_decay"}
    names = {n for n, _ in model.named_parameters()}
    assert set(groups["normal"]) | set(groups["no_weight_decay"]) == names and not set(groups["normal"]) & set(groups["no_weight_decay"])
    for name in groups["no_weight_decay"]:
        assert name.endswith("bias") or "ln_" in name or "norm" in name or "state_weight" in name or "wpe" in name or "wte" in name, name
    for name in groups["normal"]:
        assert not name.endswith(".bias"), name
    assert "transformer.h.1.sequence_mixer.state_weight" in groups["no_weight_decay"]
    torch_groups = get_torch_param_groups(model, {"lr": 1e-3, "weight_decay": 0.1}, None)
    decays = sorted(g.get("weight_decay", 0.1) for g in torch_groups)
    assert decays == [0, 0.1]
    assert sum(len(g["params"]) for g in torch_groups) == len(names)


def test_mup_parameter_groups_scale_the_learning_rate():
    from lm_engine.optimization.params_group import get_param_groups_with_names, get_torch_param_groups

    with pytest.raises(ValueError):
        get_param_groups_with_names(_tiny_model(), ParamsGroupMethod.mup)  # the model must be initialised for muP as well
    model = _tiny_model(init_method="mup", m_width=4.0)
    groups = get_param_groups_with_names(model, ParamsGroupMethod.mup)
    assert set(groups) == {"normal", "no_weight_decay", "mup"}
    assert any(name.endswith("c_fc.weight") for name in groups["mup"]) and any(name.endswith("c_attn.weight") for name in groups["mup"])
    assert not any("wte" in name for name in groups["mup"])
    torch_groups = get_torch_param_groups(model, {"lr": 1e-3, "weight_decay": 0.1}, ParamsGroupMethod.mup)
    rates = sorted({g.get("lr", 1e-3) for g in torch_groups})
    assert rates == [1e-3 / 4.0, 1e-3]


def test_metrics_tracking_dict_accumulates_and_averages():
    from lm_engine.utils.loss_dict import MetricsTrackingDict

    total = MetricsTrackingDict({})
    for step in range(4):
        total = total + {"loss": torch.tensor(float(step)), "grad_norm": 2.0}
    mean = total / 4
    assert float(mean["loss"]) == pytest.approx(1.5) and float(mean["grad_norm"]) == pytest.approx(2.0)
    assert set(mean.keys()) == {"loss", "grad_norm"}

"""Megatron-format data stack: store round trip, native index builders against their Python statement, sample
continuity, blending, sampler coverage, and the dataloader entry point."""

import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from lm_engine.data.megatron import (BlendedDataset, BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig, MegatronBatchSampler,
                                     MMapIndexedDataset, MMapIndexedDatasetBuilder, Split, get_megatron_gpt_dataloaders)
from lm_engine.data.megatron import utils as mutils
from lm_engine.data.megatron.indexed_dataset import DType, get_bin_path, get_idx_path
from lm_engine.data.megatron.merge_data import merge_files

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
EOD = 1


def _write_store(prefix: str, num_docs: int, seed: int, dtype=np.uint16, vocab: int = 1000):
    rng = np.random.RandomState(seed)
    builder = MMapIndexedDatasetBuilder(get_bin_path(prefix), dtype=dtype)
    docs = []
    for _ in range(num_docs):
        doc = np.concatenate([rng.randint(2, vocab, size=rng.randint(3, 90)), [EOD]])
        docs.append(doc)
        builder.add_item(torch.from_numpy(doc))
        builder.end_document()
    builder.finalize(get_idx_path(prefix))
    return docs


def _config(**kwargs):
    base = dict(is_built_on_rank=True, random_seed=1234, sequence_length=32, split="100,0,0")
    base.update(kwargs)
    return GPTDatasetConfig(**base)


def test_store_round_trip_and_merge(tmp_path):
    a, b, merged = (str(tmp_path / n) for n in ("a", "b", "merged"))
    docs_a, docs_b = _write_store(a, 17, 0), _write_store(b, 9, 1)
    store = MMapIndexedDataset(a)
    assert len(store) == 17 and store.index.dtype == np.uint16
    assert MMapIndexedDataset.exists(a) and not MMapIndexedDataset.exists(a + "x")
    for i, doc in enumerate(docs_a):
        assert np.array_equal(store[i], doc)
        assert np.array_equal(store.get(i, offset=1, length=2), doc[1:3])
    assert all(np.array_equal(x, y) for x, y in zip(store[3:7], docs_a[3:7]))
    assert np.array_equal(store.document_indices, np.arange(18))
    assert DType.optimal_dtype(50000) == np.uint16 and DType.optimal_dtype(128256) == np.int32

    merge_files([a, b], merged)
    both = MMapIndexedDataset(merged)
    assert len(both) == 26 and np.array_equal(both.document_indices, np.arange(27))
    for i, doc in enumerate(docs_a + docs_b):
        assert np.array_equal(both[i], doc)
    import pickle

    clone = pickle.loads(pickle.dumps(both))
    assert np.array_equal(clone[25], docs_b[-1])


def test_native_index_builders_match_python_statement(monkeypatch):
    if mutils._helpers() is None:
        pytest.skip("extension not built")
    rng = np.random.RandomState(0)
    sizes = rng.randint(1, 200, size=300).astype(np.int32)
    for dtype in (np.int32, np.int64):
        for seq, epochs in ((16, 1), (64, 3), (333, 2)):
            doc_idx = np.tile(np.arange(300, dtype=dtype), epochs)
            rng.shuffle(doc_idx)
            tokens = int(sizes.sum())
            native = mutils.build_sample_idx(sizes, doc_idx, seq, epochs, tokens)
            with monkeypatch.context() as m:
                m.setattr(mutils, "_helpers", lambda: None)
                python = mutils.build_sample_idx(sizes, doc_idx, seq, epochs, tokens)
            assert native.dtype == python.dtype == dtype and np.array_equal(native, python)
    weights = mutils.normalize([0.3, 0.5, 0.2])
    out = []
    for fake in (False, True):
        index, sample = np.zeros(1000, dtype=np.int16), np.zeros(1000, dtype=np.int64)
        with monkeypatch.context() as m:
            if fake:
                m.setattr(mutils, "_helpers", lambda: None)
            mutils.build_blending_indices(index, sample, weights, 3, 1000, False)
        out.append((index, sample))
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
    counts = np.bincount(out[0][0], minlength=3)
    assert np.abs(counts - np.array(weights) * 1000).max() <= 1


@pytest.mark.parametrize("num_samples", [20, 400])  # one epoch, several epochs
def test_gpt_dataset_samples_tile_the_token_stream(tmp_path, num_samples):
    prefix = str(tmp_path / "corpus")
    docs = _write_store(prefix, 40, 3)
    config = _config(path_to_cache=str(tmp_path / "cache"))
    store = MMapIndexedDataset(prefix)
    dataset = GPTDataset(store, np.arange(40, dtype=np.int32), num_samples, Split.train, None, config, caching_allowed=True)
    assert len(dataset) >= num_samples
    stream = np.concatenate([docs[d] for d in dataset.document_index])
    inverse = np.argsort(dataset.shuffle_index)
    seq = config.sequence_length
    for position in range(len(dataset)):
        sample = dataset[int(inverse[position])]["text"]
        assert sample.dtype == np.int64 and sample.shape == (seq + 1,)
        assert np.array_equal(sample, stream[position * seq : position * seq + seq + 1])
    assert sorted(dataset.shuffle_index.tolist()) == list(range(len(dataset)))

    # second construction must come from the cache, and without permission to write
    again = GPTDataset(store, np.arange(40, dtype=np.int32), num_samples, Split.train, None, config, caching_allowed=False)
    assert np.array_equal(again.sample_index, dataset.sample_index) and np.array_equal(again.shuffle_index, dataset.shuffle_index)
    assert len(os.listdir(tmp_path / "cache")) == 4


class _CharTokenizer:
    eod = EOD

    def convert_tokens_to_ids(self, token):
        return {"<fim_suffix>": 1001, "<fim_prefix>": 1002, "<fim_middle>": 1003, "<fim_pad>": 1004}[token]

    def detokenize(self, ids):
        return "".join(chr(int(i) + 200) for i in ids)

    def tokenize(self, text):
        return [ord(c) - 200 for c in text]


def test_fill_in_the_middle_keeps_length_and_tokens(tmp_path):
    prefix = str(tmp_path / "corpus")
    _write_store(prefix, 30, 5)
    store = MMapIndexedDataset(prefix)
    plain = GPTDataset(store, np.arange(30, dtype=np.int32), 25, Split.train, _CharTokenizer(), _config(path_to_cache=str(tmp_path / "c")), True)
    fim = GPTDataset(store, np.arange(30, dtype=np.int32), 25, Split.train, _CharTokenizer(),
                     _config(path_to_cache=str(tmp_path / "c"), fim_rate=1.0, fim_spm_rate=0.5), True)
    changed = 0
    for i in range(25):
        a, b = plain[i]["text"], fim[i]["text"]
        assert a.shape == b.shape
        assert b[0] == 1002 and np.isin(b, [1001, 1002, 1003]).sum() >= 2  # later sentinels may fall off the window
        # document boundaries stay where they were in number (the sentinels may push the last ones out of the window)
        assert (b == EOD).sum() <= (a == EOD).sum()
        ordinary = b[b < 1000]
        assert np.isin(ordinary, a).all()
        changed += int(not np.array_equal(a, b))
    assert changed == 25


def test_blended_builder_and_weights(tmp_path):
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    _write_store(a, 60, 7)
    _write_store(b, 50, 8)
    config = _config(blend=["0.7", a, "0.3", b], split="90,10,0", path_to_cache=str(tmp_path / "cache"))
    train, valid, test = BlendedMegatronDatasetBuilder(GPTDataset, [200, 20, 0], config, None).build()
    assert isinstance(train, BlendedDataset) and isinstance(valid, BlendedDataset) and test is None
    assert len(train) == sum(int(np.ceil(200 * w * 1.005)) for w in (0.7, 0.3))
    share = np.bincount(np.asarray(train.dataset_index), minlength=2) / len(train)
    assert abs(share[0] - 0.7) < 0.01
    item = train[5]
    assert item["text"].shape == (33,) and item["dataset_id"] in (0, 1)
    # train and valid come from disjoint sequence ranges of each store
    assert train.datasets[0].indexed_indices.max() < valid.datasets[0].indexed_indices.min()

    single = BlendedMegatronDatasetBuilder(GPTDataset, [50, 0, 0], _config(blend=[a], split="1,0,0", path_to_cache=str(tmp_path / "cache")), None).build()
    assert isinstance(single[0], GPTDataset) and single[1] is None and single[2] is None

    per_split = _config(blend_per_split=[[a], ["1", a, "1", b], None], split=None, path_to_cache=str(tmp_path / "cache"))
    train, valid, test = BlendedMegatronDatasetBuilder(GPTDataset, [30, 10, 5], per_split, None).build()
    assert isinstance(train, GPTDataset) and isinstance(valid, BlendedDataset) and test is None

    groups = BlendedMegatronDatasetBuilder(GPTDataset, [30, 10, 5], _config(split=None, path_to_cache=str(tmp_path / "cache")), None)
    out = groups.build_dataset_single_split([["g", "g"], ["h"]], [[a, b], [a]], [["0:0.5", "0.5:1"], ["0:1"]], [[3, 1], [1]], Split.valid)
    assert isinstance(out[0], BlendedDataset) and isinstance(out[1], GPTDataset)
    assert out[0].datasets[0].unique_identifiers["name"] == "g" and out[0].datasets[0].unique_identifiers["split"] == "0:0.5"


def test_batch_sampler_deals_disjoint_slices_and_resumes():
    total, micro, replicas = 103, 4, 3
    seen = []
    per_rank = [list(MegatronBatchSampler(total, 0, micro, replicas, r)) for r in range(replicas)]
    assert len({len(b) for b in per_rank}) == 1 and len(per_rank[0]) == total // (micro * replicas)
    for step in range(len(per_rank[0])):
        batch = sum((per_rank[r][step] for r in range(replicas)), [])
        assert batch == list(range(step * micro * replicas, (step + 1) * micro * replicas))
        seen += batch
    resumed = list(MegatronBatchSampler(total, 5 * micro * replicas, micro, replicas, 1))
    assert resumed == per_rank[1][5:]
    tail = list(MegatronBatchSampler(10, 0, 4, 2, 0, drop_last=False))
    assert tail == [[0, 1, 2, 3], [8, 9]]


def test_dataloader_entry_point_single_process(tmp_path):
    prefix = str(tmp_path / "corpus")
    _write_store(prefix, 80, 11)
    args = SimpleNamespace(
        datasets=[SimpleNamespace(class_args={"data_path": [prefix], "split": "80,20,0", "sequence_length": 16, "eval_steps": 2,
                                              "data_cache_path": str(tmp_path / "cache"), "num_workers": 0},
                                  max_input_tokens=None, max_output_tokens=None, input_format="__input__", output_format="__output__")],
        training_parameters=SimpleNamespace(micro_batch_size=4, gradient_accumulation_steps=2, num_training_steps=5, eval_interval=2),
        distributed_args=SimpleNamespace(num_pipeline_stages=1, dispatching_dataloader=False),
        random_args=SimpleNamespace(seed=42))
    train, val, test = get_megatron_gpt_dataloaders(args, None, consumed_samples=0)
    first = next(train)["text"]
    assert first.shape == (4, 17) and first.dtype == torch.int64
    assert len(val) == 1 and next(val[0])["text"].shape == (4, 17) and test == [None]
    resumed, _, _ = get_megatron_gpt_dataloaders(args, None, consumed_samples=4)
    second = next(train)["text"]
    assert torch.equal(next(resumed)["text"], second)


_REF_CHILD = r"""
import sys, types, numpy as np
repo, ref, prefix, out = sys.argv[1:5]
sys.path.insert(0, repo)
from lm_engine.ops.build import load_extension
helpers = load_extension(build_if_missing=False)
for name in [k for k in sys.modules if k == "lm_engine" or k.startswith("lm_engine.")]:
    del sys.modules[name]
sys.path.remove(repo)
sys.path.insert(0, ref)
sys.modules["helpers"] = helpers
from lm_engine.data.megatron.indexed_dataset import MMapIndexedDataset
from lm_engine.data.megatron.gpt_dataset import GPTDataset
from lm_engine.data.megatron.blended_megatron_dataset_config import GPTDatasetConfig
from lm_engine.data.megatron.utils import Split
store = MMapIndexedDataset(prefix)
result = {}
for n in (20, 400):
    config = GPTDatasetConfig(is_built_on_rank=True, random_seed=1234, sequence_length=32, blend=[prefix], split="100,0,0", path_to_cache=out + f"_cache{n}")
    ds = GPTDataset(store, np.arange(len(store), dtype=np.int32), n, Split.train, None, config, True)
    result[f"doc{n}"], result[f"sample{n}"], result[f"shuffle{n}"] = np.array(ds.document_index), np.array(ds.sample_index), np.array(ds.shuffle_index)
    result[f"text{n}"] = np.stack([ds[i]["text"] for i in range(n)])
    result[f"hash{n}"] = np.frombuffer(ds.unique_description_hash.encode(), dtype=np.uint8)
np.savez(out, **result)
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_indices_and_samples_match_reference(tmp_path):
    if mutils._helpers() is None:
        pytest.skip("extension not built")
    prefix = str(tmp_path / "corpus")
    _write_store(prefix, 40, 3)
    out = str(tmp_path / "ref.npz")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    done = subprocess.run([sys.executable, "-c", _REF_CHILD, ROOT, REF, prefix, out], cwd=str(tmp_path), env=env, timeout=600, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]
    ref = np.load(out)
    store = MMapIndexedDataset(prefix)
    for n in (20, 400):
        config = _config(blend=[prefix], path_to_cache=str(tmp_path / f"mine{n}"))
        ds = GPTDataset(store, np.arange(40, dtype=np.int32), n, Split.train, None, config, True)
        assert ds.unique_description_hash == bytes(ref[f"hash{n}"]).decode()
        assert np.array_equal(ds.document_index, ref[f"doc{n}"])
        assert np.array_equal(ds.sample_index, ref[f"sample{n}"])
        assert np.array_equal(ds.shuffle_index, ref[f"shuffle{n}"])
        assert np.array_equal(np.stack([ds[i]["text"] for i in range(n)]), ref[f"text{n}"])


def test_stand_alone_dataloader_tool(tmp_path):
    """``lm_engine.cli.megatron_dataloader``: the loaders without the rest of the engine (library call and command line), weighted
    blend of two stores, resumption by the number of consumed samples."""
    import subprocess

    from lm_engine.cli.megatron_dataloader import build_dataloaders

    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    _write_store(a, 80, 3)
    _write_store(b, 60, 4)
    common = dict(data_path=[0.7, a, 0.3, b], split="90,10,0", sequence_length=16, micro_batch_size=4, num_training_steps=6,
                  data_cache_path=str(tmp_path / "cache"), eval_during_training=True, eval_interval=3, num_workers=0)
    train, validation, test = build_dataloaders(**common)
    first, second = next(train)["text"], next(train)["text"]
    assert first.shape == (4, 17) and len(validation) == 1 and test == []
    resumed, _, _ = build_dataloaders(**common, consumed_samples=4)
    assert torch.equal(next(resumed)["text"], second)

    done = subprocess.run([sys.executable, "-m", "lm_engine.cli.megatron_dataloader", "--data-path", "0.7", a, "0.3", b, "--split", "90,10,0",
                           "--sequence-length", "16", "--micro-batch-size", "4", "--num-training-steps", "6", "--cache", str(tmp_path / "cache"),
                           "--show", "2"], cwd=ROOT, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert "batch 1: text (4, 17)" in done.stdout and f"first tokens {first[0, :8].tolist()}" in done.stdout


_CONVERT = r"""
import sys
sys.path.insert(0, sys.argv[1])
from lm_engine.data.megatron.preprocess_data import convert_file
class Tokenizer:
    vocab_size = 1000
    eos_token_id = 1
    def encode(self, text):
        return [2 + sum(map(ord, word)) % 900 for word in text.split()]
convert_file(Tokenizer(), sys.argv[2], sys.argv[3], workers=1, chunk_size=4)
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lm_engine")), reason="reference is not installed under baseline/_ref")
def test_converted_store_is_byte_identical_to_the_reference_s(tmp_path):
    """An arrow file of token lists converted to a ``.bin/.idx`` store by this package and by the reference: the same bytes in
    both files (the reference's converter reaches only its arrow branch: its jsonl branch opens the wrong name)."""
    import subprocess

    import pyarrow as pa

    schema = pa.schema([pa.field("tokens", pa.uint32())])
    source = str(tmp_path / "in.arrow")
    with pa.ipc.new_file(source, schema) as writer:
        for i in range(20):
            writer.write(pa.record_batch([pa.array([(i * 7 + j) % 900 + 2 for j in range(3 + i % 6)], type=pa.uint32())], schema))
    for which, package in (("theirs", REF), ("mine", ROOT)):
        done = subprocess.run([sys.executable, "-c", _CONVERT, package, source, str(tmp_path / which)], cwd=str(tmp_path),
                              env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
    for suffix in ("_text.bin", "_text.idx"):
        mine, theirs = (tmp_path / f"mine{suffix}").read_bytes(), (tmp_path / f"theirs{suffix}").read_bytes()
        assert len(mine) > 100 and mine == theirs, suffix

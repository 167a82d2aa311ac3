"""Streaming loader over arrow shards: coverage of an epoch across ranks, packing, weighted sampling, exact resume, and
resume on another number of ranks."""

import os

import pyarrow as pa
import pytest
import torch

from lm_engine.data.ibm import (ArrowHandler, BufferDataset, CheckpointDataset, PreloadBufferDataset, SamplingDataset,
                                ScalableShardDataset, StreamingDocDataset, build_experimental_data_loader, train_config)

EOS, BOS = 0, 1


def _write_dataset(root, name, n_files, docs_per_file, first_id):
    """Every document is [id, id, ..., id] (random length) so that documents can be recognised in the stream."""
    os.makedirs(os.path.join(root, name), exist_ok=True)
    schema = pa.schema([pa.field("tokens", pa.uint32())])
    doc_id, lengths = first_id, {}
    g = torch.Generator().manual_seed(first_id)
    for f in range(n_files):
        with pa.ipc.new_file(os.path.join(root, name, f"shard_{f}.arrow"), schema) as writer:
            for _ in range(docs_per_file):
                n = int(torch.randint(3, 40, (1,), generator=g))
                writer.write(pa.record_batch([pa.array([doc_id] * n, type=pa.uint32())], schema))
                lengths[doc_id] = n
                doc_id += 1
    return lengths


def _documents(chunks):
    """Split a stream of chunks at EOS and return the document ids with their body lengths."""
    out, current = [], []
    for chunk in chunks:
        for token in chunk:
            if token == EOS:
                body = [t for t in current if t != BOS]
                out.append((body[0], len(body)))
                current = []
            else:
                current.append(token)
    return out


def _take(iterator, n):
    return [next(iterator) for _ in range(n)]


def test_ranks_cover_every_document_once_per_epoch(tmp_path):
    root = str(tmp_path / "data")
    lengths = _write_dataset(root, "a", n_files=3, docs_per_file=17, first_id=100)
    seen = []
    for rank in range(4):
        reader = StreamingDocDataset(os.path.join(root, "a"), rank, 4, ArrowHandler(), EOS, bos_token=BOS, max_chunksize=16)
        reader.setup()
        it = iter(reader)
        docs, pending = [], []
        while len(docs) < reader.docs_per_epoch:
            chunk = next(it)
            assert len(chunk) <= 16
            pending.append(chunk)
            if chunk[-1] == EOS:
                docs += _documents(pending)
                pending = []
        assert reader.epochs_seen == 0
        seen += docs
    assert sorted(d for d, _ in seen) == sorted(lengths)
    assert all(lengths[d] == n for d, n in seen)


def _stack(root, rank, world, window=8, shards=8, weights=(3.0, 1.0)):
    reader = StreamingDocDataset(root, rank, world, ArrowHandler(), EOS, bos_token=BOS, max_chunksize=64)
    stack = ScalableShardDataset(reader, EOS, n_logical_shards=shards)
    stack = SamplingDataset(root, stack, EOS, datasets=["a", "b"], weights=list(weights))
    stack = BufferDataset(stack, 33, pack_hard=True)
    return PreloadBufferDataset(stack, window)


def test_packing_weights_and_exact_resume(tmp_path):
    root = str(tmp_path / "data")
    _write_dataset(root, "a", 2, 40, 100)
    _write_dataset(root, "b", 2, 40, 1000)
    stack = _stack(root, 0, 2)
    it = iter(stack)
    first = _take(it, 50)
    assert all(len(line) == 33 for line in first)
    tokens = [t for line in first for t in line if t not in (EOS, BOS)]
    share_a = sum(1 for t in tokens if t < 1000) / len(tokens)
    assert 0.65 < share_a < 0.85  # weights 3 : 1

    state = stack.state_dict()
    expected = _take(it, 30)
    fresh = _stack(root, 0, 2)
    fresh.load_state_dict([state], sharded_input=True)
    assert _take(iter(fresh), 30) == expected


def test_resume_on_fewer_ranks_keeps_every_stream_position(tmp_path):
    root = str(tmp_path / "data")
    _write_dataset(root, "a", 2, 40, 100)
    _write_dataset(root, "b", 2, 40, 1000)
    stacks = [_stack(root, r, 2) for r in range(2)]
    iterators = [iter(s) for s in stacks]
    for it in iterators:
        _take(it, 25)
    states = [s.state_dict() for s in stacks]
    positions = {}
    for s in stacks:
        for name, child in zip(s.dataset.dataset.datasets, s.dataset.dataset.data):
            for logical, reader in zip(child.logicals_owned, child.data):
                positions[(name, logical)] = (reader.docs_seen, reader.tokens_seen)

    merged = _stack(root, 0, 1)
    merged.load_state_dict(states)
    assert len(merged.buffer) == 16  # the shuffle windows of both old ranks were merged ...
    it = iter(merged)
    _take(it, 12)  # ... drain back to the window size, then the streams are read again
    assert len(merged.buffer) == 8
    restored = {}
    for name, child in zip(merged.dataset.dataset.datasets, merged.dataset.dataset.data):
        assert child.logicals_owned == list(range(8))
        for logical, reader in zip(child.logicals_owned, child.data):
            restored[(name, logical)] = (reader.docs_seen, reader.tokens_seen)
    # every logical stream continues from where its previous owner left it (the one line pulled may have advanced some)
    assert set(restored) == set(positions)
    assert all(restored[k][0] >= positions[k][0] and restored[k][1] >= positions[k][1] for k in positions)
    assert any(restored[k] != positions[k] for k in positions)


def test_loader_factory_and_auto_checkpoint(tmp_path):
    root = str(tmp_path / "data")
    _write_dataset(root, "a", 2, 30, 100)
    _write_dataset(root, "b", 1, 30, 1000)
    cfg = train_config(dict(dataset_path=root, datasets="a,b", weights="1,1", seq_len=16, batch_size=4, eos_token=EOS, bos_token=BOS,
                            logical_shards=4, shuffle_window=4, num_workers=0, enable_checkpoint=True,
                            checkpoint_folder=str(tmp_path / "ckpt"), checkpoint_interval=3, file_type="arrow", col_name="tokens"))
    loader = build_experimental_data_loader(cfg, None, rank=0, world_size=1)
    batches = _take(loader, 8)
    assert all(b.shape == (4, 17) and b.dtype == torch.int64 for b in batches)
    saved = sorted(os.listdir(tmp_path / "ckpt"))
    assert saved == ["step-3", "step-6"] and os.listdir(tmp_path / "ckpt" / "step-6") == ["loader_state_0.pth"]
    # a new loader picks up the latest state and continues with the batch that followed it
    resumed = build_experimental_data_loader(cfg, None, rank=0, world_size=1)
    assert torch.equal(next(resumed), batches[6])


# the same scenario text runs against the reference (child process) and against this package (here)
_REFERENCE_SCENARIO = r"""
import copy
import os
import torch
import tempfile
from lm_engine.data.ibm import (ArrowHandler, BufferDataset, PreloadBufferDataset, PreprocessDataset, SamplingDataset, ScalableShardDataset,
                                StreamingDocDataset, build_experimental_data_loader, train_config)
from lm_engine.utils import ProcessGroupManager

def plain(value):
    if isinstance(value, torch.Tensor):
        return value.tolist()
    if isinstance(value, dict):
        return {key: plain(item) for key, item in value.items()}
    if isinstance(value, (list, tuple)):
        return [plain(item) for item in value]
    return value

def take(iterator, n):
    return [plain(next(iterator)) for _ in range(n)]

def scenario(root):
    out = {}
    for rank in range(3):
        d = StreamingDocDataset(os.path.join(root, "a"), rank, 3, ArrowHandler(), 0, bos_token=1, max_chunksize=16, seed=7)
        d.setup()
        out[f"stream_rank{rank}"] = take(iter(d), 60)
    d = StreamingDocDataset(os.path.join(root, "b"), 0, 1, ArrowHandler(), 0, max_chunksize=1000, min_length=5, seed=3)
    d.setup()
    out["stream_long_chunks"] = take(iter(d), 50)
    for rank in range(2):
        d = ScalableShardDataset(StreamingDocDataset(os.path.join(root, "a"), rank, 2, ArrowHandler(), 0, max_chunksize=16, seed=5), 0, n_logical_shards=8)
        d.setup()
        out[f"scalable_rank{rank}"] = take(iter(d), 60)
    d = SamplingDataset(root, StreamingDocDataset(root, 0, 1, ArrowHandler(), 0, max_chunksize=16, seed=9), 0, datasets=["a", "b"], weights=[3, 1])
    d.setup()
    out["sampling"] = take(iter(d), 80)
    for hard in (True, False):
        d = BufferDataset(StreamingDocDataset(os.path.join(root, "a"), 0, 1, ArrowHandler(), 0, max_chunksize=16, seed=7), 24, pack_hard=hard,
                          bos_token=1, eos_token=0, pad_token=2)
        d.setup()
        out[f"buffer_hard{int(hard)}"] = take(iter(d), 30)
    d = PreloadBufferDataset(StreamingDocDataset(os.path.join(root, "a"), 0, 1, ArrowHandler(), 0, max_chunksize=16, seed=7), 10)
    d.setup()
    out["preload"] = take(iter(d), 40)

    # a position saved in the middle of a document, and what follows it
    def reader():
        made = BufferDataset(StreamingDocDataset(os.path.join(root, "a"), 0, 1, ArrowHandler(), 0, bos_token=1, max_chunksize=8, seed=11), 20, pack_hard=True)
        made.setup()
        return made
    first = reader()
    stream = iter(first)
    out["before_saving"] = take(stream, 23)
    out["saved_state"] = plain(first.state_dict())
    out["after_saving"] = take(stream, 40)
    second = reader()
    second.load_state_dict([copy.deepcopy(out["saved_state"])])  # the reference extends a loaded buffer in place
    out["after_loading"] = take(iter(second), 40)

    # automatic saving: directory names, files, and the stream of a second instance that finds them
    import tempfile
    from lm_engine.data.ibm import CheckpointDataset
    folder = tempfile.mkdtemp()
    def saver():
        made = CheckpointDataset(BufferDataset(StreamingDocDataset(os.path.join(root, "b"), 0, 1, ArrowHandler(), 0, max_chunksize=8, seed=2), 12, pack_hard=True),
                                 folder, 5, steps_per_batch=2)
        made.setup()
        return made
    first = saver()
    out["autosave_stream"] = take(iter(first), 27)
    out["autosave_tree"] = sorted((name, sorted(os.listdir(os.path.join(folder, name)))) for name in os.listdir(folder))
    second = saver()
    out["autosave_resumed_step"] = second.step
    out["autosave_resumed_stream"] = take(iter(second), 7)

    # four ranks save, two and eight ranks load: the streams of the logical shards move with their positions
    def stack(rank, world):
        made = StreamingDocDataset(os.path.join(root, "a"), rank, world, ArrowHandler(), 0, max_chunksize=16, seed=5)
        made = PreloadBufferDataset(BufferDataset(ScalableShardDataset(made, 0, n_logical_shards=8), 20, pack_hard=True), 6)
        made.setup()
        return made
    states = []
    for rank in range(4):
        saved = stack(rank, 4)
        stream = iter(saved)
        out[f"rescale_before_rank{rank}"] = take(stream, 15)
        states.append(saved.state_dict())
    for world in (2, 8):
        for rank in range(world):
            loaded = stack(rank, world)
            loaded.load_state_dict(copy.deepcopy(states))
            logical = loaded.dataset.dataset
            out[f"rescale_to{world}_rank{rank}"] = [plain(logical.n_docs_remaining),
                                                     [[r.rank, r.docset_index, r.chunk_index, r.lcg_state] for r in logical.data],
                                                     take(iter(loaded), 25 if world == 2 else 6)]

    # the whole stack as the training entry point builds it
    cfg = train_config(dict(dataset_path=root, datasets="a,b", weights="2,1", drop_tokens="", bos_token=1, eos_token=0, file_type="arrow", col_name="tokens",
                            logical_shards=8, seq_len=31, batch_size=3, num_workers=0, enable_checkpoint=False, checkpoint_model_weights_only=False))
    for rank in range(2):
        with ProcessGroupManager.set_dummy_data_parallel_rank(rank), ProcessGroupManager.set_dummy_data_parallel_world_size(2):
            loader = build_experimental_data_loader(cfg, None)
            out[f"loader_rank{rank}"] = take(loader, 12)
    return out


def job_scenario(root):
    out = {}
    folder = tempfile.mkdtemp()
    def cfg():
        return train_config(dict(dataset_path=root, datasets="a,b", weights="2,1", drop_tokens="", bos_token=1, eos_token=0, file_type="arrow", col_name="tokens",
                                 logical_shards=8, seq_len=31, batch_size=2, num_workers=1, enable_checkpoint=True, checkpoint_model_weights_only=False,
                                 checkpoint_folder=folder, checkpoint_interval=4, gradient_accumulation_steps=1))
    loaders = []
    for rank in range(4):
        with ProcessGroupManager.set_dummy_data_parallel_rank(rank), ProcessGroupManager.set_dummy_data_parallel_world_size(4):
            loaders.append(build_experimental_data_loader(cfg(), None))
    firsts = [[] for _ in loaders]
    for step in range(6):  # all ranks advance together, as the ranks of a job do
        for rank, loader in enumerate(loaders):
            firsts[rank].append(next(loader).tolist())
    for rank in range(4):
        out[f"first_rank{rank}"] = firsts[rank]
    del loaders
    out["tree"] = sorted((name, sorted(os.listdir(os.path.join(folder, name)))) for name in os.listdir(folder))
    resumed = []
    for rank in range(2):
        with ProcessGroupManager.set_dummy_data_parallel_rank(rank), ProcessGroupManager.set_dummy_data_parallel_world_size(2):
            resumed.append(build_experimental_data_loader(cfg(), None))
    lines = [[] for _ in resumed]
    for step in range(5):
        for rank, loader in enumerate(resumed):
            lines[rank].append(next(loader).tolist())
    for rank in range(2):
        out[f"resumed_rank{rank}"] = lines[rank]
    out["tree_after"] = sorted((name, sorted(os.listdir(os.path.join(folder, name)))) for name in os.listdir(folder))
    out["folder"] = folder
    return out
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "lm_engine")),
                    reason="reference is not installed under baseline/_ref")
def test_streams_saved_positions_and_the_full_stack_equal_the_reference(tmp_path):
    """Token for token what the reference's classes of the same names produce from the same shard files: the document
    streams of three ranks (with and without a start token, short and long chunks, a minimum length), logical shards on two
    ranks, weighted sampling of two datasets, hard and soft packing into lines, the shuffle window, the position saved in the
    middle of a document (the same state dict) and the stream after loading it, automatic saving, the states of four ranks loaded
    by two and by eight ranks (counts and positions of the logical shards, the lines that follow), and the batches of the whole
    stack as the training entry point builds it, on two data-parallel ranks."""
    import json
    import subprocess
    import sys

    reference = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    root = str(tmp_path / "data")
    _write_dataset(root, "a", n_files=3, docs_per_file=17, first_id=100)
    _write_dataset(root, "b", n_files=2, docs_per_file=11, first_id=500)
    child = ("import json, sys\nsys.path.insert(0, sys.argv[1])\nexec(sys.argv[2])\n"
             "json.dump(dict(scenario(sys.argv[3]), job=job_scenario(sys.argv[3])), open(sys.argv[4], 'w'))\n")
    out = tmp_path / "theirs.json"
    done = subprocess.run([sys.executable, "-c", child, reference, _REFERENCE_SCENARIO, root, str(out)], cwd=str(tmp_path),
                          env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), timeout=600, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]
    theirs = json.loads(out.read_text())
    scope: dict = {}
    exec(_REFERENCE_SCENARIO, scope)
    mine = json.loads(json.dumps(scope["scenario"](root)))
    their_job = theirs.pop("job")
    assert set(mine) == set(theirs) and len(theirs) == 34
    for key in theirs:
        assert mine[key] == theirs[key], key
    assert mine["after_loading"] == mine["after_saving"]
    assert mine["autosave_resumed_step"] == 10 and mine["autosave_resumed_stream"] == mine["autosave_stream"][20:27]

    # the whole stack with automatic saving as a job runs it: four ranks (one loader worker each) advance together and save,
    # two ranks find the states and go on. Same batches and same files on both sides; and the files the reference wrote
    # are read here (two ranks again) to the batches the reference itself resumed with.
    my_job = json.loads(json.dumps(scope["job_scenario"](root)))
    their_folder = their_job.pop("folder")
    my_job.pop("folder")
    assert my_job == their_job and [name for name, _ in their_job["tree"]] == ["step-4"]
    import shutil

    from lm_engine.data.ibm import build_experimental_data_loader, train_config

    for name in os.listdir(their_folder):  # back to what the two resuming ranks found: the states of the four ranks
        if name != "step-4":
            shutil.rmtree(os.path.join(their_folder, name))
    cfg = train_config(dict(dataset_path=root, datasets="a,b", weights="2,1", drop_tokens="", bos_token=1, eos_token=0, file_type="arrow",
                            col_name="tokens", logical_shards=8, seq_len=31, batch_size=2, num_workers=1, enable_checkpoint=True,
                            checkpoint_model_weights_only=False, checkpoint_folder=their_folder, checkpoint_interval=4,
                            gradient_accumulation_steps=1))
    loaders = [build_experimental_data_loader(cfg, None, rank=rank, world_size=2) for rank in range(2)]
    lines = [[], []]
    for _ in range(5):
        for rank, loader in enumerate(loaders):
            lines[rank].append(next(loader).tolist())
    assert lines[0] == their_job["resumed_rank0"] and lines[1] == their_job["resumed_rank1"]

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
    saved = sorted(os.listdir(tmp_path / "ckpt" / "checkpoints"))
    assert saved == ["step-3_ckp", "step-6_ckp"]
    # a new loader picks up the latest state and continues with the batch that followed it
    resumed = build_experimental_data_loader(cfg, None, rank=0, world_size=1)
    assert torch.equal(next(resumed), batches[6])

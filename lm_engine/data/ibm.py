"""Stateful, rescalable streaming dataloader over tokenised shard files (arrow / parquet).

Parity: lm_engine/data/ibm.py:21-1472 (the IBM/FMS loader). The pipeline is a stack of iterable datasets, each of which
can report and restore its position so that a run resumes mid-epoch, also on a different number of ranks:

    StreamingDocDataset     documents of this rank's share of the shard files, in a per-epoch pseudo-random order, cut
                            into chunks of at most ``max_chunksize`` tokens with bos/eos delimiters
    ScalableShardDataset    ``n_logical_shards`` independent streams dealt to the ranks; a restart on another world size
                            re-deals the streams (with their positions) instead of the files
    SamplingDataset         one stream per sub-dataset, drawn so that the tokens seen follow the given weights
    BufferDataset           packs the chunks into lines of exactly ``seq_len + 1`` tokens
    PreloadBufferDataset    shuffles lines inside a window
    PreprocessDataset       maps every line (here: to a LongTensor)
    CheckpointDataset       saves the whole stack's state every ``interval`` batches and reloads the latest one

State dictionaries are per (loader worker) rank; :meth:`load_state_dict` takes the list of all saved ranks' states and
picks / re-deals what belongs to this rank.
"""

from __future__ import annotations

import csv
import logging
import math
import os
import random
import time
from copy import deepcopy
from typing import Any, Callable

import torch
import torch.utils.data as data

from ..utils import ProcessGroupManager, log_rank_0


class train_config:
    """Attribute bag built from the dataset's ``class_args``."""

    def __init__(self, d: dict | None = None) -> None:
        for key, value in (d or {}).items():
            setattr(self, key, value)

    def set(self, key: str, value) -> None:
        setattr(self, key, value)

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({', '.join(f'{k}={v!r}' for k, v in self.__dict__.items())})"


def _shard_partition(items: list, rank: int, world: int) -> list:
    """Contiguous chunk ``rank`` of ``world`` (sizes differ by at most one)."""
    return items[(rank * len(items)) // world : ((rank + 1) * len(items)) // world]


def _shard_inclusive(items: list, rank: int, world: int) -> list:
    """Like :func:`_shard_partition` but including items of which this rank owns only a fraction."""
    return items[math.floor(len(items) * rank / world) : math.ceil(len(items) * (rank + 1) / world)]


def _get_latest(directory: str, qualifier: Callable[[str], bool] = lambda path: True) -> str | None:
    """The entry ``<prefix>-<number>...`` with the largest number, or None."""
    if not os.path.isdir(directory):
        return None
    candidates = [os.path.join(directory, name) for name in os.listdir(directory)]
    candidates = [c for c in candidates if qualifier(c)]
    if not candidates:
        return None
    return max(candidates, key=lambda path: int(os.path.basename(path).split("-")[1].split("_")[0]))


# ----------------------------------------------------------------------------------------------------------------------
# stateful dataset base classes
class _StatefulDataset(data.IterableDataset):
    """``state_params``: scalars that describe a position and are only valid for the same world size;
    ``reshard_params``: lists that can be re-dealt to another world size."""

    def __init__(self, datapath: str | None, rank: int, worldsize: int) -> None:
        assert 0 <= rank < worldsize
        self.datapath = datapath
        self.rank, self.worldsize = rank, worldsize
        self.local_worldsize = -1
        self.state_params: list[str] = []
        self.reshard_params: list[str] = []
        self.is_setup = False
        self.coordinates_final = False  # True: a parent layer already folded the loader worker into (rank, worldsize)
        self.load_worldsize = worldsize

    def setup(self) -> None:
        """Deferred initialisation, run in the loader worker: folds the worker id into the rank."""
        if self.is_setup:
            return
        self.is_setup = True
        info = None if self.coordinates_final else data.get_worker_info()
        if self.coordinates_final:
            self.local_worldsize = max(self.local_worldsize, 1)
        elif info is not None:
            self.local_worldsize = info.num_workers
            self.worldsize *= info.num_workers
            self.rank = self.rank * info.num_workers + info.id
        else:
            self.local_worldsize = 1

    def statename(self, name: str) -> str:
        return f"{type(self).__name__}.{name}"

    def state_dict(self) -> dict:
        self.setup()
        # copies: the live lists keep changing while the iteration goes on
        return {self.statename(name): deepcopy(getattr(self, name)) for name in self.state_params + self.reshard_params}

    def _reshard(self, lists: list[list]) -> list:
        """Concatenate the saved ranks' lists and take this rank's share."""
        flat = [item for part in lists for item in part]
        return _shard_partition(flat, self.rank, self.worldsize)

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        """``state_dicts``: the states of all saved ranks (or, with ``sharded_input``, already only those this rank
        overlaps). Scalars are restored only when the world size is unchanged; lists are always re-dealt."""
        self.setup()
        self.load_worldsize = len(state_dicts) if not sharded_input else self.load_worldsize
        mine = state_dicts if sharded_input else _shard_inclusive(state_dicts, self.rank, self.worldsize)
        if self.load_worldsize == self.worldsize and len(mine) == 1:
            for name in self.state_params:
                setattr(self, name, mine[0][self.statename(name)])
        for name in self.reshard_params:
            if self.load_worldsize == self.worldsize and len(mine) == 1:
                setattr(self, name, mine[0][self.statename(name)])
            else:
                all_lists = [sd[self.statename(name)] for sd in state_dicts]
                setattr(self, name, self._reshard(all_lists))
        return mine

    def load_from_path(self, path: str) -> None:
        files = sorted((f for f in os.listdir(path) if f.startswith("loader_state_")), key=lambda f: int(f.split("_")[-1].split(".")[0]))
        assert files, f"no loader state under {path}"
        self.setup()
        self.load_worldsize = len(files)
        wanted = _shard_inclusive(files, self.rank, self.worldsize)
        self.load_state_dict([torch.load(os.path.join(path, f), weights_only=False) for f in wanted], sharded_input=True)

    def save_to_path(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        torch.save(self.state_dict(), os.path.join(path, f"loader_state_{self.rank}.pth"))


class _WrapperDataset(_StatefulDataset):
    """A layer around another stateful dataset; state calls recurse."""

    def __init__(self, dataset: _StatefulDataset) -> None:
        super().__init__(dataset.datapath, dataset.rank, dataset.worldsize)
        self.dataset = dataset

    def setup(self) -> None:
        if not self.is_setup:
            super().setup()
            self.dataset.setup()

    def state_dict(self) -> dict:
        self.setup()
        return {**self.dataset.state_dict(), **super().state_dict()}

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        self.setup()
        mine = super().load_state_dict(state_dicts, sharded_input)
        self.dataset.load_worldsize = self.load_worldsize
        self.dataset.load_state_dict(mine, sharded_input=True)
        return mine


# ----------------------------------------------------------------------------------------------------------------------
# shard file formats
class _ShardFileHandler:
    def is_legal(self, filepath: str) -> bool:
        return os.path.isfile(filepath)

    def open(self, path: str):
        raise NotImplementedError

    def length(self, path: str) -> int:
        raise NotImplementedError

    def get(self, reader, index: int, drop_tokens: set):
        raise NotImplementedError

    def slice(self, doc, index: int, n_pull: int) -> list:
        raise NotImplementedError


class ArrowHandler(_ShardFileHandler):
    """Pre-tokenised documents, one record batch per document, token ids in column ``col_name``."""

    def __init__(self, col_name: str = "tokens") -> None:
        self.col_name = col_name

    def is_legal(self, filepath: str) -> bool:
        return filepath.endswith(".arrow")

    def open(self, path: str):
        import pyarrow as pa

        return pa.ipc.open_file(pa.memory_map(path))

    def length(self, path: str) -> int:
        return self.open(path).num_record_batches

    def get(self, reader, index: int, drop_tokens: set):
        doc = reader.get_batch(index)[self.col_name]
        if len(doc) > 0 and doc[0].as_py() in drop_tokens:
            doc = doc.slice(1, len(doc) - 1)
        if len(doc) > 0 and doc[-1].as_py() in drop_tokens:
            doc = doc.slice(0, len(doc) - 1)
        return doc

    def slice(self, doc, index: int, n_pull: int) -> list:
        return doc.slice(index, n_pull).to_pylist()


class ParquetHandler(_ShardFileHandler):
    """Raw text documents in column ``col_name``, tokenised on the fly."""

    def __init__(self, tokenizer, col_name: str = "text") -> None:
        self.tokenizer = tokenizer
        self.col_name = col_name

    def is_legal(self, filepath: str) -> bool:
        return filepath.endswith(".parquet")

    def open(self, path: str):
        import pyarrow.parquet as pq

        return pq.read_pandas(path, columns=[self.col_name], partitioning=None)[self.col_name]

    def length(self, path: str) -> int:
        import pyarrow.parquet as pq

        return pq.read_metadata(path).num_rows

    def get(self, reader, index: int, drop_tokens: set):
        doc = self.tokenizer(str(reader[index]))["input_ids"]
        if len(doc) > 0 and doc[0] in drop_tokens:
            doc = doc[1:]
        if len(doc) > 0 and doc[-1] in drop_tokens:
            doc = doc[:-1]
        return doc

    def slice(self, doc: list, index: int, n_pull: int) -> list:
        return doc[index : index + n_pull]


_handler_map = {"arrow": ArrowHandler, "hf_parquet": ParquetHandler}


# ----------------------------------------------------------------------------------------------------------------------
class StreamingDocDataset(_StatefulDataset):
    """Streams the documents of ``datapath/<dataset>`` (shard files, possibly nested) that fall to this rank.

    The documents of all files form one numbered range; rank ``r`` of ``w`` owns the contiguous share
    ``[r / w, (r + 1) / w)`` of it, so files may be split between ranks. Within an epoch the owned documents are
    visited in the order of a full-period linear congruential generator (no shuffle array is kept); a document is
    emitted as chunks of at most ``max_chunksize`` tokens, the first starting with ``bos`` (when set) and the last
    ending with ``delimiter_token``. Document counts come from ``meta/*.csv`` (columns: path, documents, tokens) when
    present, otherwise from the files themselves.
    """

    def __init__(self, datapath: str, rank: int, worldsize: int, filehandler: _ShardFileHandler, delimiter_token: Any,
                 bos_token: Any | None = None, strip_tokens: set | None = None, seed: int = 42, min_length: int = 1,
                 max_chunksize: int = 1024, verbose: bool = False) -> None:
        super().__init__(datapath, rank, worldsize)
        self.filehandler = filehandler
        self.eos, self.bos = delimiter_token, bos_token
        self.drop = set(strip_tokens or ())
        self.seed, self.min_length, self.chunksize, self.verbose = seed, min_length, max_chunksize, verbose
        self.docset: list[tuple[str, int, int]] = []  # (file, first doc, last doc) inclusive, owned by this rank
        self.dataset = ""
        self.docs_per_epoch = 0
        # position
        self.docset_index = 0  # documents of the current epoch already started
        self.chunk_index = -1  # last chunk emitted of the current document (-1: none)
        self.epochs_seen = -1
        self.tokens_seen = 0
        self.docs_seen = 0
        self.percent_seen = 0.0
        self.lcg_state = seed + rank
        self.state_params = ["dataset", "docset_index", "chunk_index", "epochs_seen", "tokens_seen", "docs_seen", "percent_seen", "lcg_state"]

    # -- discovery -------------------------------------------------------------------------------------------------------
    def _document_counts(self, root: str, files: list[str]) -> dict[str, int]:
        meta = os.path.join(os.path.dirname(root.rstrip("/")), "meta")
        counts: dict[str, int] = {}
        if os.path.isdir(meta):
            for name in os.listdir(meta):
                if not name.endswith(".csv"):
                    continue
                with open(os.path.join(meta, name)) as handle:
                    for row in csv.DictReader(handle):
                        path = row.get("dataset/filename") or row.get("path") or ""
                        for f in files:
                            if path.endswith(os.path.relpath(f, os.path.dirname(root.rstrip("/")))) or path.endswith(os.path.basename(f)):
                                counts[f] = int(row.get("documents") or row.get("docs") or 0)
        for f in files:
            if f not in counts or counts[f] <= 0:
                counts[f] = self.filehandler.length(f)
        return counts

    def setup(self) -> None:
        if self.is_setup:
            return
        super().setup()
        root = self.datapath
        self.dataset = os.path.basename(root.rstrip("/")) if not self.dataset else self.dataset
        files = sorted(os.path.join(folder, name) for folder, _, names in os.walk(root) for name in names
                       if self.filehandler.is_legal(os.path.join(folder, name)))
        assert files, f"no shard files of the expected type under {root}"
        counts = self._document_counts(root, files)
        total = sum(counts[f] for f in files)
        first = (total * self.rank) // self.worldsize
        last = (total * (self.rank + 1)) // self.worldsize  # exclusive
        cursor = 0
        for f in files:
            lo, hi = max(first, cursor), min(last, cursor + counts[f])
            if hi > lo:
                self.docset.append((f, lo - cursor, hi - cursor - 1))
            cursor += counts[f]
        self.docs_per_epoch = sum(hi - lo + 1 for _, lo, hi in self.docset)
        assert self.docs_per_epoch > 0, f"rank {self.rank} of {self.worldsize} owns no document of {root}"
        if self.epochs_seen < 0 and self.docset_index == 0:
            self.lcg_state = self.seed + self.rank  # fresh start: the stream depends on the final (worker-folded) rank

    # -- order -----------------------------------------------------------------------------------------------------------
    def _locate(self, index: int) -> tuple[str, int]:
        for f, lo, hi in self.docset:
            span = hi - lo + 1
            if index < span:
                return f, lo + index
            index -= span
        raise IndexError(index)

    def _next_random_document(self) -> int:
        """Full-period LCG modulo the next power of two, skipping values outside the range: a permutation of
        ``range(docs_per_epoch)`` per period, continued across epochs from the saved state."""
        modulus = 1 << max(int(math.ceil(math.log2(max(self.docs_per_epoch, 2)))), 1)
        while True:
            self.lcg_state = (5 * self.lcg_state + 2 * self.seed + 1) % modulus  # a = 1 mod 4, c odd: full period
            if self.lcg_state < self.docs_per_epoch:
                return self.lcg_state

    def _chunks(self, doc) -> int:
        length = len(doc) + (1 if self.bos is not None else 0) + 1
        return max(math.ceil(length / self.chunksize), 1)

    def _chunk(self, doc, j: int, n_chunks: int) -> list:
        """Chunk ``j`` of the delimited document ``[bos] doc eos``."""
        offset = 1 if self.bos is not None else 0
        start = j * self.chunksize
        stop = min((j + 1) * self.chunksize, len(doc) + offset + 1)
        out: list = []
        if j == 0 and self.bos is not None:
            out.append(self.bos)
        body_lo, body_hi = max(start - offset, 0), min(stop - offset, len(doc))
        if body_hi > body_lo:
            out.extend(self.filehandler.slice(doc, body_lo, body_hi - body_lo))
        if j == n_chunks - 1:
            out.append(self.eos)
        return out

    def __iter__(self):
        self.setup()
        reader, open_path = None, None
        resume_doc = self.docset_index > 0 and self.chunk_index >= 0  # mid-document restart
        while True:
            if self.docset_index == 0 and not resume_doc:
                self.epochs_seen += 1
            while self.docset_index < self.docs_per_epoch or resume_doc:
                if resume_doc:
                    local, first_chunk = self._current_doc, self.chunk_index + 1
                    resume_doc = False
                else:
                    local, first_chunk = self._next_random_document(), 0
                    self._current_doc = local
                    self.docset_index += 1
                path, row = self._locate(local)
                if path != open_path:
                    reader, open_path = self.filehandler.open(path), path
                doc = self.filehandler.get(reader, row, self.drop)
                if len(doc) < self.min_length:
                    continue
                n_chunks = self._chunks(doc)
                for j in range(first_chunk, n_chunks):
                    chunk = self._chunk(doc, j, n_chunks)
                    self.chunk_index = j
                    self.tokens_seen += len(chunk)
                    if j == n_chunks - 1:
                        self.docs_seen += 1
                        self.chunk_index = -1
                        self.percent_seen = self.docs_seen * 100.0 / self.docs_per_epoch
                    yield chunk
            self.docset_index = 0

    def state_dict(self) -> dict:
        out = super().state_dict()
        out[self.statename("_current_doc")] = getattr(self, "_current_doc", 0)
        return out

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        self.setup()
        assert self.load_worldsize == self.worldsize or sharded_input, (
            "StreamingDocDataset alone cannot change the number of ranks; wrap it in ScalableShardDataset")
        mine = super().load_state_dict(state_dicts, sharded_input)
        if len(mine) == 1 and self.statename("_current_doc") in mine[0]:
            self._current_doc = mine[0][self.statename("_current_doc")]
        return mine


class ScalableShardDataset(_WrapperDataset):
    """``n_logical_shards`` copies of the wrapped reader, each owning ``1 / n_logical_shards`` of the documents, dealt
    evenly to the ranks. What a checkpoint stores is the position of every logical shard, so a restart on any world size
    that divides ``n_logical_shards`` continues every stream where it stopped. Streams of a rank are drawn at random in
    proportion to the documents they have left in the current pass, which keeps them in step."""

    def __init__(self, dataset: StreamingDocDataset, delimiter_token: Any, n_logical_shards: int = 2048, verbose: bool = False) -> None:
        super().__init__(dataset)
        assert n_logical_shards % self.worldsize == 0, f"world size {self.worldsize} must divide n_logical_shards {n_logical_shards}"
        self.total_shards = n_logical_shards
        self.delimiter = delimiter_token
        self.verbose = verbose
        self.data: list[StreamingDocDataset] = []
        self.logicals_owned: list[int] = []
        self.n_logicals = 0
        self.n_docs_remaining: list[int] = []
        self.generator = None
        self.current_reader = None  # stream that is in the middle of a document
        self.logical_shard_states: list[dict] | None = None
        self.g_state = None
        self.state_params = ["current_reader", "g_state"]
        self.reshard_params = ["n_docs_remaining", "logical_shard_states"]

    def setup(self) -> None:
        if self.is_setup:
            return
        _StatefulDataset.setup(self)
        n = self.total_shards // self.worldsize
        self.n_logicals = n
        self.logicals_owned = list(range(n * self.rank, n * (self.rank + 1)))
        for index in self.logicals_owned:
            reader = deepcopy(self.dataset)
            reader.worldsize, reader.rank = self.total_shards, index
            reader.local_worldsize, reader.coordinates_final, reader.is_setup = 1, True, False
            reader.lcg_state = reader.seed + index
            reader.setup()
            self.data.append(reader)
        self.n_docs_remaining = [d.docs_per_epoch for d in self.data]
        self.generator = torch.Generator().manual_seed(self.rank)

    def __iter__(self):
        self.setup()
        if self.logical_shard_states is not None:  # restored positions, one per owned stream
            for reader, state in zip(self.data, self.logical_shard_states):
                reader.load_worldsize = reader.worldsize
                reader.load_state_dict([state], sharded_input=True)
            self.logical_shard_states = None
        if self.g_state is not None:
            self.generator.set_state(self.g_state)
        iterators = [iter(d) for d in self.data]
        while True:
            if self.current_reader is not None:
                index = self.current_reader
            else:
                if sum(self.n_docs_remaining) == 0:
                    self.n_docs_remaining = [d.docs_per_epoch for d in self.data]
                    self.generator.manual_seed(self.rank)
                weights = torch.tensor(self.n_docs_remaining, dtype=torch.float)
                index = int(torch.multinomial(weights, 1, generator=self.generator))
                self.current_reader = index
            chunk = next(iterators[index])
            if chunk[-1] == self.delimiter:  # document finished: choose afresh next time
                self.n_docs_remaining[index] -= 1
                self.current_reader = None
            yield chunk

    def state_dict(self) -> dict:
        self.setup()
        self.g_state = self.generator.get_state()
        self.logical_shard_states = [d.state_dict() for d in self.data]
        out = _StatefulDataset.state_dict(self)
        self.logical_shard_states = None
        return out

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        self.setup()
        return _StatefulDataset.load_state_dict(self, state_dicts, sharded_input)


class SamplingDataset(_WrapperDataset):
    """One copy of the wrapped dataset per sub-directory of ``datapath``; the next document always comes from the
    sub-dataset whose share of the tokens produced so far lags its weight the most."""

    def __init__(self, datapath: str, dataset: _StatefulDataset, delimiter_token: Any, datasets: list[str] | None = None,
                 weights: list[float] | None = None, verbose: bool = False) -> None:
        super().__init__(dataset)
        self.datapath = datapath
        self.delimiter = delimiter_token
        self.verbose = verbose
        self.datasets = list(datasets) if datasets is not None else sorted(
            d for d in os.listdir(datapath) if os.path.isdir(os.path.join(datapath, d)) and d != "meta")
        assert self.datasets, "no sub-datasets found"
        weights = [1.0] * len(self.datasets) if weights is None else [float(w) for w in weights]
        assert len(weights) == len(self.datasets) and all(w > 0 for w in weights)
        self.weights = [w / sum(weights) for w in weights]
        self.data: list[_StatefulDataset] = []
        self.tokens_seen = [0] * len(self.datasets)
        self.current_iterator = -1
        self.state_params = ["tokens_seen", "current_iterator"]

    def setup(self) -> None:
        if self.is_setup:
            return
        _StatefulDataset.setup(self)
        for name in self.datasets:
            child = deepcopy(self.dataset)
            _repath(child, os.path.join(self.datapath, name), self.rank, self.worldsize, self.local_worldsize)
            child.setup()
            self.data.append(child)

    def __iter__(self):
        self.setup()
        iterators = [iter(d) for d in self.data]
        while True:
            if self.current_iterator == -1:
                total = sum(self.tokens_seen) + 1e-9
                lag = [w - seen / total for w, seen in zip(self.weights, self.tokens_seen)]
                self.current_iterator = max(range(len(lag)), key=lag.__getitem__)
            chunk = next(iterators[self.current_iterator])
            self.tokens_seen[self.current_iterator] += len(chunk)
            if chunk[-1] == self.delimiter:
                self.current_iterator = -1
            yield chunk

    def state_dict(self) -> dict:
        self.setup()
        out = {}
        for name, child in zip(self.datasets, self.data):
            out.update({f"{name}.{k}": v for k, v in child.state_dict().items()})
        out.update(_StatefulDataset.state_dict(self))
        return out

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        self.setup()
        mine = _StatefulDataset.load_state_dict(self, state_dicts, sharded_input)
        for name, child in zip(self.datasets, self.data):
            prefix = name + "."
            child.load_worldsize = self.load_worldsize
            child.load_state_dict([{k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)} for sd in mine], sharded_input=True)
        return mine


def _repath(dataset: _StatefulDataset, datapath: str, rank: int, worldsize: int, local_worldsize: int) -> None:
    """Point a (not yet set up) dataset stack at another directory with already folded rank coordinates."""
    node = dataset
    while node is not None:
        node.datapath, node.rank, node.worldsize, node.local_worldsize = datapath, rank, worldsize, local_worldsize
        node.is_setup, node.coordinates_final = False, True
        node = getattr(node, "dataset", None) if isinstance(getattr(node, "dataset", None), _StatefulDataset) else None


class BufferDataset(_WrapperDataset):
    """Re-cuts the stream of variable-length chunks into lines of exactly ``seq_len`` tokens. ``pack_hard`` splits
    chunks across lines; otherwise a chunk that does not fit starts a new line and the old one is padded."""

    def __init__(self, dataset: _StatefulDataset, seq_len: int, pack_hard: bool, bos_token=None, eos_token=None, pad_token=None) -> None:
        super().__init__(dataset)
        self.len = seq_len
        self.pack_hard = pack_hard
        self.bos, self.eos, self.pad = bos_token, eos_token, pad_token
        if not pack_hard:
            assert pad_token is not None, "soft packing pads lines: a pad token is needed"
        self.buffer: list = []
        self.state_params = ["buffer"]

    def __iter__(self):
        self.setup()
        source = iter(self.dataset)
        while True:
            if self.pack_hard:
                while len(self.buffer) < self.len:
                    self.buffer = self.buffer + list(next(source))
                line, self.buffer = self.buffer[: self.len], self.buffer[self.len :]
            else:
                line = self.buffer
                self.buffer = []
                while True:
                    chunk = list(next(source))[: self.len]
                    if len(line) + len(chunk) > self.len:
                        self.buffer = chunk
                        break
                    line = line + chunk
                line = line + [self.pad] * (self.len - len(line))
            if self.bos is not None and line[0] != self.bos:
                line = [self.bos] + line[:-1]
            if self.eos is not None and line[-1] != self.eos:
                line = line[:-1] + [self.eos]
            yield line


class PreloadBufferDataset(_WrapperDataset):
    """Shuffle inside a window: keeps ``window_size`` lines, emits a random one and refills its place. After a restart
    on fewer ranks the re-dealt windows are larger than ``window_size`` and drain back to it."""

    def __init__(self, dataset: _StatefulDataset, window_size: int) -> None:
        super().__init__(dataset)
        assert window_size > 1
        self.window_size = window_size
        self.g_state = None
        self.generator = torch.Generator().manual_seed(self.rank)
        self.buffer: list[list] = []
        self.state_params = ["g_state"]
        self.reshard_params = ["buffer"]

    def __iter__(self):
        self.setup()
        source = iter(self.dataset)
        if self.g_state is not None:
            self.generator.set_state(self.g_state)
        while True:
            while len(self.buffer) < self.window_size:
                self.buffer.append(next(source))
            index = int(torch.randint(len(self.buffer), (1,), generator=self.generator))
            out = self.buffer[index]
            if len(self.buffer) > self.window_size:  # drain an oversized (re-dealt) window
                self.buffer[index] = self.buffer[-1]
                self.buffer.pop()
            else:
                self.buffer[index] = next(source)
            yield out

    def state_dict(self) -> dict:
        self.g_state = self.generator.get_state()
        return super().state_dict()


class PreprocessDataset(_WrapperDataset):
    """Applies ``aug_fn`` to every item."""

    def __init__(self, dataset: _StatefulDataset, aug_fn: Callable) -> None:
        super().__init__(dataset)
        self.aug_fn = aug_fn

    def __iter__(self):
        self.setup()
        for item in iter(self.dataset):
            yield self.aug_fn(item)


class CheckpointDataset(_WrapperDataset):
    """Saves the state of the whole stack to ``<save_path>/checkpoints/step-<n>_ckp/`` every ``interval`` batches of
    ``steps_per_batch`` items, and loads the latest one under ``load_path`` at the first iteration."""

    def __init__(self, dataset: _StatefulDataset, load_path: str, interval: int, steps_per_batch: int = 1, save_path: str = "") -> None:
        super().__init__(dataset)
        self.interval = interval
        self.spb = max(int(steps_per_batch), 1)
        self.load_path = load_path
        self.path = os.path.join(save_path or load_path, "checkpoints")
        self.step = 0
        self.ministep = 0
        self.state_params = ["step", "ministep"]

    def setup(self) -> None:
        if not self.is_setup:
            super().setup()
            self.load_from_path(self.load_path)

    def __iter__(self):
        self.setup()
        for item in iter(self.dataset):
            yield item
            self.ministep += 1
            if self.ministep == self.spb:
                self.ministep = 0
                self.step += 1
                if self.step % self.interval == 0:
                    self.save_to_path(os.path.join(self.path, f"step-{self.step}_ckp"))

    def _latest(self, path: str) -> str | None:
        """A directory of loader states, or the newest ``step-<n>_ckp`` below ``path`` / ``path/checkpoints``."""
        if not path or not os.path.isdir(path):
            return None
        if any(name.startswith("loader_state_") for name in os.listdir(path)):
            return path
        for root in (path, os.path.join(path, "checkpoints")):
            latest = _get_latest(root, lambda p: os.path.isdir(p) and os.path.basename(p).startswith("step-") and p.endswith("_ckp")
                                 ) if os.path.isdir(root) else None
            if latest is not None and any(name.startswith("loader_state_") for name in os.listdir(latest)):
                return latest
        return None

    def load_from_path(self, path: str) -> None:
        latest = self._latest(path)
        if latest is None:
            log_rank_0(logging.INFO, f"no dataloader checkpoint under {path}: starting from the beginning")
            return
        started = time.time()
        self.dataset.load_from_path(latest)
        state_file = os.path.join(latest, f"checkpointer_{self.rank}.pth")
        if os.path.isfile(state_file):
            own = torch.load(state_file, weights_only=False)
            self.step, self.ministep = own["step"], own["ministep"]
        else:
            self.step = int(os.path.basename(latest).split("-")[1].split("_")[0])
        log_rank_0(logging.INFO, f"dataloader state loaded from {latest} in {time.time() - started:.1f} s (step {self.step})")

    def save_to_path(self, path: str) -> None:
        self.dataset.save_to_path(path)
        torch.save({"step": self.step, "ministep": self.ministep}, os.path.join(path, f"checkpointer_{self.rank}.pth"))


# ----------------------------------------------------------------------------------------------------------------------
def parse_data_args(datas, weights):
    def split(x):
        if isinstance(x, str):
            return [item.strip() for item in x.split(",")]
        if isinstance(x, (list, tuple)):
            return list(x)
        if isinstance(x, (int, float)):
            return [x]
        raise ValueError(f"arg input {x} cannot be parsed.")

    datas = split(datas) if datas is not None else None
    weights = [float(w) for w in split(weights)] if weights is not None else None
    return datas, weights


def build_experimental_data_loader(cfg: train_config, tokenizer, rank: int | None = None, world_size: int | None = None):
    """The full stack for causal language modelling; yields ``LongTensor [batch_size, seq_len + 1]``."""
    datasets, weights = parse_data_args(cfg.get("datasets"), cfg.get("weights"))
    rank = ProcessGroupManager.get_data_parallel_rank() if rank is None else rank
    world_size = ProcessGroupManager.get_data_parallel_world_size() if world_size is None else world_size

    drop = [int(x.strip()) for x in str(cfg.get("drop_tokens", "")).split(",") if x.strip()]
    bos, eos = cfg.get("bos_token", -1), cfg.eos_token
    drop += [bos, eos]
    file_type = cfg.get("file_type", "arrow")
    assert file_type in _handler_map, f"File type {file_type} is not recognized ({list(_handler_map)})"
    if file_type == "hf_parquet":
        assert tokenizer is not None, "raw text shards need a tokenizer"
        handler = ParquetHandler(tokenizer, cfg.get("col_name", "text"))
    else:
        handler = _handler_map[file_type](cfg.get("col_name", "tokens"))

    stack = StreamingDocDataset(cfg.dataset_path, rank, world_size, handler, eos, bos_token=None if bos == -1 else bos,
                                strip_tokens=set(drop), min_length=3, seed=cfg.get("seed", 42),
                                max_chunksize=cfg.get("max_chunksize", 1024))
    stack = ScalableShardDataset(stack, eos, n_logical_shards=cfg.get("logical_shards", 2048))
    stack = SamplingDataset(cfg.dataset_path, stack, eos, datasets=datasets, weights=weights)
    stack = BufferDataset(stack, cfg.seq_len + 1, pack_hard=True)
    stack = PreloadBufferDataset(stack, cfg.get("shuffle_window", 10000))
    stack = PreprocessDataset(stack, torch.LongTensor)
    num_workers = cfg.get("num_workers", 1)
    if cfg.get("enable_checkpoint", False) and not cfg.get("checkpoint_model_weights_only", False):
        stack = CheckpointDataset(stack, cfg.checkpoint_folder, cfg.checkpoint_interval,
                                  cfg.batch_size * cfg.get("gradient_accumulation_steps", 1) / max(num_workers, 1))
    return iter(data.DataLoader(stack, num_workers=num_workers, batch_size=cfg.batch_size))


def get_ibm_dataloaders(args, tokenizer):
    assert len(args.datasets) == 1
    cfg = train_config(args.datasets[0].class_args)
    cfg.set("batch_size", args.training_parameters.micro_batch_size)
    cfg.set("seq_len", cfg.sequence_length)
    cfg.set("checkpoint_interval", args.save_args.save_interval)
    cfg.set("gradient_accumulation_steps", args.training_parameters.gradient_accumulation_steps)
    loader = _TextBatches(build_experimental_data_loader(cfg, tokenizer))
    return loader, [], []


class _TextBatches:
    """Wraps every batch as ``{"text": batch}``, the form the pretraining wrapper takes."""

    def __init__(self, iterator) -> None:
        self.iterator = iterator

    def __iter__(self):
        return self

    def __next__(self):
        return {"text": next(self.iterator)}

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
picks / re-deals what belongs to this rank. From the same shard files and arguments every layer emits, token for token,
what the reference's class of the same name emits, and saves the same position.
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
        """This rank's share of the saved ranks' lists. ``lists`` are those of the saved ranks that this rank overlaps
        (``_shard_inclusive`` of all of them), all of one length: positions are counted over the lists of ALL saved ranks
        and shifted by what lies left of the first list given."""
        length = len(lists[0])
        assert all(len(part) == length for part in lists), "the saved ranks hold lists of different lengths"
        skipped = math.floor(self.load_worldsize * self.rank / self.worldsize) * length  # items of the saved ranks not given
        total = self.load_worldsize * length
        first, last = int(total * self.rank / self.worldsize) - skipped, int(total * (self.rank + 1) / self.worldsize) - skipped
        return [lists[i // length][i % length] for i in range(first, last)]

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        """``state_dicts``: the states of all saved ranks (or, with ``sharded_input``, already only those this rank
        overlaps). Scalars are restored only when the world size is unchanged; lists are always re-dealt."""
        self.setup()
        self.load_worldsize = len(state_dicts) if not sharded_input else self.load_worldsize
        mine = state_dicts if sharded_input else _shard_inclusive(state_dicts, self.rank, self.worldsize)
        if self.load_worldsize == self.worldsize and len(mine) == 1:
            for name in self.state_params + self.reshard_params:
                setattr(self, name, mine[0][self.statename(name)])
        else:
            for name in self.reshard_params:
                setattr(self, name, self._reshard([sd[self.statename(name)] for sd in mine]))
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

        names = pq.read_metadata(path).schema.names
        column = self.col_name
        if column not in names:  # the usual names of the text column in hub datasets
            found = [name for name in ("text", "content", "contents") if name in names]
            assert len(found) == 1, f"{path}: no column {self.col_name!r} and {len(found)} of text / content / contents"
            column = found[0]
        return pq.read_pandas(path, columns=[column], partitioning=None)[column]

    def length(self, path: str) -> int:
        import pyarrow.parquet as pq

        return pq.read_metadata(path).num_rows

    def get(self, reader, index: int, drop_tokens: set):
        # whole documents are tokenised before they are cut: a bound on the text keeps a pathological one affordable
        doc = self.tokenizer(str(reader[index])[:128_000])["input_ids"]
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
    """Streams the documents of ``datapath`` (shard files, possibly nested) that fall to this rank.

    Partition: the shard files, in sorted order, are laid end to end by size (the ``size`` column of ``../meta/*counts*.csv``
    when there is one, else the file sizes); rank ``r`` of ``w`` owns the stretch ``[r / w, (r + 1) / w]`` of that line, and
    of every file it touches the documents whose numbers fall inside the matching fraction. Order: the owned file pieces
    are shuffled once (seeded by ``seed + rank``) and read one after the other, so a file is opened once per epoch; within
    a piece the documents come in the order of a full-period linear congruential generator, no index array is kept.
    A document is emitted as chunks of at most ``max_chunksize`` tokens, the first starting with ``bos`` (when set) and the
    last ending with ``delimiter_token``. The stream, and the saved position (``docset_index``, ``chunk_index``,
    ``lcg_state``), are those of the reference's class of the same name (lm_engine/data/ibm.py:742-1086).
    """

    def __init__(self, datapath: str, rank: int, worldsize: int, filehandler: _ShardFileHandler, delimiter_token: Any,
                 bos_token: Any | None = None, strip_tokens: set | None = None, seed: int = 42, min_length: int = 1,
                 max_chunksize: int = 1024, verbose: bool = False) -> None:
        super().__init__(datapath, rank, worldsize)
        assert max_chunksize > 0, "max_chunksize must be positive"
        self.filehandler = filehandler
        self.eos, self.bos = delimiter_token, bos_token
        self.drop = set(strip_tokens or ())
        self.seed, self.min_length, self.chunksize, self.verbose = seed, min_length, max_chunksize, verbose
        self.docset: list[tuple[str, int, int]] = []  # (file relative to datapath, first doc, last doc) inclusive
        self.dataset = ""
        self.docs_per_epoch = 0
        # position: the document of the epoch that is being read, its last chunk handed out, the generator state before it
        self.docset_index = 0
        self.chunk_index = -1
        self.lcg_state = 0
        # statistics
        self.epochs_seen = -1
        self.tokens_seen = 0
        self.docs_seen = 0
        self.percent_seen = 0.0
        self.state_params = ["dataset", "docset_index", "chunk_index", "epochs_seen", "tokens_seen", "docs_seen", "percent_seen", "lcg_state"]

    # -- discovery -------------------------------------------------------------------------------------------------------
    def _metadata(self, parent: str, dataset: str) -> tuple[dict[str, int], dict[str, int]]:
        """``(sizes, documents)`` per file (relative to the dataset directory) from the first ``*counts*.csv`` under
        ``parent/meta``; empty dicts when there is none. Rows are keyed by ``.../<dataset>/<file>``."""
        folder = os.path.join(parent, "meta")
        tables = [name for name in os.listdir(folder) if "counts" in name and "csv" in name] if os.path.isdir(folder) else []
        sizes: dict[str, int] = {}
        documents: dict[str, int] = {}
        if not tables:
            return sizes, documents
        marker = f"/{dataset}/"
        with open(os.path.join(folder, tables[0])) as handle:
            for row in csv.DictReader(handle):
                path = row["dataset/filename"]
                at = path.rfind(marker)
                if at < 0:
                    continue
                key = path[at + len(marker):]
                documents[key] = int(row["documents"])
                if row.get("size") not in (None, ""):
                    sizes[key] = int(row["size"])
        return sizes, documents

    def setup(self) -> None:
        if self.is_setup:
            return
        super().setup()
        root = self.datapath
        parent, dataset = os.path.split(root.rstrip("/"))
        self.dataset = dataset
        names = sorted(os.path.join(folder, name)[len(root.rstrip("/")) + 1:] for folder, _, files in os.walk(root) for name in files
                       if self.filehandler.is_legal(os.path.join(folder, name)))
        assert names, f"no shard files of the expected type under {root}"
        sizes, documents = self._metadata(parent, dataset)
        weights = [sizes[name] for name in names] if sizes else [os.path.getsize(os.path.join(root, name)) for name in names]
        total = sum(weights)
        shares = [weight / total for weight in weights]
        lo, hi = self.rank / self.worldsize, (self.rank + 1) / self.worldsize
        cursor, owned = 0, []
        for name, share in zip(names, shares):
            if cursor <= hi and cursor + share >= lo:
                owned.append((name, min(max((lo - cursor) / share, 0), 1), min(max((hi - cursor) / share, 0), 1)))
            cursor += share
        self.docset = []
        for name, first_fraction, last_fraction in owned:
            count = documents[name] if documents else self.filehandler.length(os.path.join(root, name))
            first, last = round(count * first_fraction), round(count * last_fraction) - 1
            if last >= first:
                self.docset.append((name, first, last))
        self.docs_per_epoch = sum(last - first + 1 for _, first, last in self.docset)
        # the order of the pieces and the generator both depend on the final (worker-folded) rank
        random.Random(self.seed + self.rank).shuffle(self.docset)
        self.lcg_state = self.seed + self.rank

    # -- order -----------------------------------------------------------------------------------------------------------
    def _piece_of(self, index: int) -> tuple[str, int, int]:
        """``(file, documents in the piece, first document)`` of the piece that holds document ``index`` of the epoch."""
        for name, first, last in self.docset:
            span = last - first + 1
            if index < span:
                return name, span, first
            index -= span
        raise IndexError(index)

    def _draw(self, size: int) -> int:
        """Next value below ``size`` of the generator ``x -> 5 x + c`` modulo the next power of two (``c`` odd, so the period
        is full: ``size`` consecutive draws visit every document of a piece once), from the saved state."""
        modulus = 2 ** math.ceil(math.log2(size))
        increment = (self.rank + self.seed) * 2 + 1
        state = self.lcg_state
        while True:
            state = (5 * state + increment) % modulus
            if state < size:
                return state

    def _chunk(self, doc, j: int, n_chunks: int) -> list:
        """Chunk ``j`` of the delimited document ``[bos] doc eos``."""
        start, pull = j * self.chunksize, self.chunksize
        if self.bos is not None:
            if j == 0:
                pull -= 1
            else:
                start -= 1
        out = self.filehandler.slice(doc, start, pull)
        self.tokens_seen += len(out)
        if self.bos is not None and j == 0:
            out = [self.bos] + out
        if j == n_chunks - 1:
            out = out + [self.eos]
        return out

    def _read(self, index: int, files: dict, first_chunk: int, stop_chunk: int | None):
        """Chunks ``[first_chunk, stop_chunk)`` (to the end of the document when ``stop_chunk`` is None) of document ``index``
        of the epoch; the generator's return value is the state that the draw for this document left."""
        name, span, first = self._piece_of(index)
        drawn = self._draw(span)
        path = os.path.join(self.datapath, name)
        if files.get("path") != path:
            files["path"], files["reader"] = path, self.filehandler.open(path)  # one open file at a time
        doc = self.filehandler.get(files["reader"], first + drawn, self.drop)
        if len(doc) == 0:
            return drawn
        length = len(doc) + (1 if self.bos is None else 2)
        if length >= self.min_length:
            n_chunks = math.ceil(length / self.chunksize)
            for j in range(first_chunk, n_chunks if stop_chunk is None else stop_chunk):
                self.chunk_index = j
                if stop_chunk is None and j == n_chunks - 1:
                    self.docs_seen += 1
                    self.percent_seen = self.docs_seen * 100 / (self.docs_per_epoch + 1e-9)
                yield self._chunk(doc, j, n_chunks)
        return drawn

    def __iter__(self):
        self.setup()
        # where the (possibly restored) position points: a pass visits every document once, starting there
        start_doc, start_state, skipped = self.docset_index, self.lcg_state, self.chunk_index + 1
        files: dict = {}
        while True:
            for step in range(self.docs_per_epoch):
                index = (start_doc + step) % self.docs_per_epoch
                if index == 0:
                    self.epochs_seen += 1
                self.docset_index = index
                self.lcg_state = yield from self._read(index, files, skipped if step == 0 else 0, None)
            # the chunks of the first document that were handed out before the restart close the pass
            self.docset_index, self.lcg_state = start_doc, start_state
            yield from self._read(start_doc, files, 0, skipped)

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        self.setup()
        assert self.load_worldsize == self.worldsize or sharded_input, (
            "StreamingDocDataset alone cannot change the number of ranks; wrap it in ScalableShardDataset")
        name = self.dataset
        mine = super().load_state_dict(state_dicts, sharded_input)
        assert name == self.dataset, f"the saved position belongs to dataset {self.dataset}, not {name}"
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
        iterators = [iter(d) for d in self.data]
        while True:
            if self.current_reader is not None:
                index = self.current_reader
            else:
                weights = torch.tensor(self.n_docs_remaining, dtype=torch.float)
                index = int(torch.multinomial(weights, 1, generator=self.generator))
                self.current_reader = index
            chunk = next(iterators[index])
            if chunk[-1] == self.delimiter:  # document finished: choose afresh next time
                self.n_docs_remaining[index] -= 1
                self.current_reader = None
                if sum(self.n_docs_remaining) == 0:
                    # the pass is over: refilled before the chunk leaves, so that a saved state never holds an exhausted
                    # count (re-dealt to another number of ranks it would starve its streams)
                    self.n_docs_remaining = [d.docs_per_epoch for d in self.data]
                    self.generator.manual_seed(self.rank)
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
        mine = _StatefulDataset.load_state_dict(self, state_dicts, sharded_input)
        if self.g_state is not None:
            self.generator.set_state(self.g_state)
        # the positions of the owned streams, applied at once: a state saved right after loading must hold them
        for reader, state in zip(self.data, self.logical_shard_states or []):
            reader.load_worldsize = reader.worldsize
            reader.load_state_dict([state], sharded_input=True)
        self.logical_shard_states = None
        return mine


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
        """The states of the sub-dataset stacks as a list under ``sample_iterator_states`` (the reference's layout,
        lm_engine/data/ibm.py:1351-1356), beside this layer's own counters."""
        self.setup()
        out = {self.statename("sample_iterator_states"): [child.state_dict() for child in self.data]}
        out.update(_StatefulDataset.state_dict(self))
        return out

    def load_state_dict(self, state_dicts: list[dict], sharded_input: bool = False) -> list[dict]:
        self.setup()
        mine = _StatefulDataset.load_state_dict(self, state_dicts, sharded_input)
        key = self.statename("sample_iterator_states")
        for index, (name, child) in enumerate(zip(self.datasets, self.data)):
            child.load_worldsize = self.load_worldsize
            if all(key in sd for sd in mine):
                parts = [sd[key][index] for sd in mine]
            else:  # states written before the list layout: the sub-dataset's keys carry its name as a prefix
                prefix = name + "."
                parts = [{k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)} for sd in mine]
            child.load_state_dict(parts, sharded_input=True)
        return mine


def _repath(dataset: _StatefulDataset, datapath: str, rank: int, worldsize: int, local_worldsize: int) -> None:
    """Point a (not yet set up) dataset stack at another directory with already folded rank coordinates."""
    node = dataset
    while node is not None:
        node.datapath, node.rank, node.worldsize, node.local_worldsize = datapath, rank, worldsize, local_worldsize
        node.is_setup, node.coordinates_final = False, True
        node = getattr(node, "dataset", None) if isinstance(getattr(node, "dataset", None), _StatefulDataset) else None


class BufferDataset(_WrapperDataset):
    """Re-cuts the stream of variable-length chunks into lines of ``seq_len`` tokens without losing a token. Chunks are
    pulled until the line would overflow. ``pack_hard``: the overflowing chunk is split across the line boundary; a token
    that has to give way to the delimiter at the end of a line opens the next line. Otherwise the chunk that does not fit
    opens the next line and the current one is closed with the delimiter and padded. A line that does not start with
    ``bos_token`` gets one. Same lines as the reference's class (lm_engine/data/ibm.py:646-739)."""

    def __init__(self, dataset: _StatefulDataset, seq_len: int, pack_hard: bool, bos_token=None, eos_token=None, pad_token=None) -> None:
        super().__init__(dataset)
        self.len = seq_len
        self.pack_hard = pack_hard
        self.bos, self.eos, self.pad = bos_token, eos_token, pad_token
        if not pack_hard:
            assert pad_token is not None, "soft packing pads lines: a pad token is needed"
        self.buffer: list = []
        self.state_params = ["buffer"]

    def _line(self, source) -> list:
        held, pending = list(self.buffer), []
        while len(held) + len(pending) < self.len:  # `pending`: the last chunk pulled, not yet part of the line
            held = held + pending
            pending = list(next(source))
        if self.bos is not None and (not held or held[0] != self.bos):
            held = [self.bos] + held
        if len(held) < self.len and not self.pack_hard:
            if self.eos is not None and held and held[-1] != self.eos:
                held = held + [self.eos]
            self.buffer = pending
            return held if self.pad is None else held + [self.pad] * (self.len - len(held))
        if len(held) < self.len:
            held, pending = held + pending, []
        line, rest = held[: self.len], held[self.len :]
        if self.eos is not None and line[-1] != self.eos:
            rest = [line[-1]] + rest
            line[-1] = self.eos
        self.buffer = rest + pending
        return line

    def __iter__(self):
        self.setup()
        source = iter(self.dataset)
        while True:
            yield self._line(source)


class PreloadBufferDataset(_WrapperDataset):
    """Shuffle inside a window of ``window_size`` lines: a random line of the window is emitted and its place refilled.
    The window grows by one line per step until it is full (so the first lines come out almost in order, as in the
    reference's class, lm_engine/data/ibm.py:570-643). After a restart on fewer ranks the re-dealt windows are larger than
    ``window_size`` and drain back to it."""

    def __init__(self, dataset: _StatefulDataset, window_size: int) -> None:
        super().__init__(dataset)
        assert window_size > 1, "a window of one line does not shuffle"
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
            if len(self.buffer) < self.window_size:
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
    """Saves the state of the whole stack to ``<save_path>/step-<n>/loader_state_<rank>.pth`` every ``interval`` batches of
    ``steps_per_batch`` items (the reference's layout, lm_engine/data/ibm.py:440-567), and at the first iteration loads the
    newest such directory: one in the save directory wins over one under ``load_path``. Directories written by earlier
    versions of this class (``checkpoints/step-<n>_ckp``) are still found."""

    def __init__(self, dataset: _StatefulDataset, load_path: str, interval: int, steps_per_batch: int = 1, save_path: str = "") -> None:
        super().__init__(dataset)
        self.interval = interval
        self.spb = max(int(steps_per_batch), 1)
        self.load_path = load_path
        self.path = save_path or load_path
        self.step = 0
        self.ministep = 0

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
                    self.save_to_path(os.path.join(self.path, f"step-{self.step}"))

    @staticmethod
    def _holds_loader_states(path: str) -> bool:
        return os.path.isdir(path) and any("loader" in name for name in os.listdir(path))

    def _latest(self, path: str) -> str | None:
        """``path`` itself when it holds loader states, else the ``step-<n>`` directory with the largest ``n`` below ``path``
        (or below ``path/checkpoints``) if that one holds loader states."""
        if not path or not os.path.isdir(path):
            return None
        if self._holds_loader_states(path):
            return path
        for root in (path, os.path.join(path, "checkpoints")):
            latest = _get_latest(root, lambda p: os.path.basename(p).startswith("step-"))
            if latest is not None and self._holds_loader_states(latest):
                return latest
        return None

    def load_from_path(self, path: str) -> None:
        latest = self._latest(self.path) or self._latest(path)
        if latest is None:
            log_rank_0(logging.INFO, f"no dataloader checkpoint under {self.path} or {path}: starting from the beginning")
            return
        started = time.time()
        self.dataset.load_from_path(latest)
        name = os.path.basename(latest.rstrip("/"))
        if name.startswith("step-"):
            self.step = int(name.split("-")[1].split("_")[0])
        log_rank_0(logging.INFO, f"dataloader state loaded from {latest} in {time.time() - started:.1f} s (step {self.step})")

    def save_to_path(self, path: str) -> None:
        started = time.time()
        self.dataset.save_to_path(path)
        log_rank_0(logging.INFO, f"dataloader state saved to {path} in {time.time() - started:.1f} s")


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

"""Memory-mapped token store in the Megatron ``.bin`` / ``.idx`` format.

Parity: lm_engine/data/megatron/indexed_dataset.py:26-616 (same on-disk format, so existing tokenised corpora load
unchanged and files written here load there).

``<prefix>.bin``  the tokens of every sequence back to back, one fixed dtype.
``<prefix>.idx``  little endian: 9-byte magic, u64 version (1), u8 dtype code, u64 sequence count, u64 document count,
                  int32 lengths[sequences], int64 byte offsets[sequences], int64 document boundaries[documents]
                  (sequence indices, starting with 0), optionally int8 modes[sequences] for multimodal stores.
"""

from __future__ import annotations

import os
import shutil
import struct
from enum import Enum

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_VERSION = 1


class DType(Enum):
    uint8 = 1
    int8 = 2
    int16 = 3
    int32 = 4
    int64 = 5
    float64 = 6
    float32 = 7
    uint16 = 8

    @classmethod
    def code_from_dtype(cls, dtype) -> int:
        return cls[np.dtype(dtype).name].value

    @classmethod
    def dtype_from_code(cls, code: int):
        return getattr(np, cls(code).name)

    @staticmethod
    def size(key) -> int:
        if isinstance(key, int):
            return np.dtype(DType.dtype_from_code(key)).itemsize
        return np.dtype(key).itemsize

    @staticmethod
    def optimal_dtype(cardinality: int | None):
        """Smallest token dtype for a vocabulary of ``cardinality`` entries."""
        return np.uint16 if cardinality is not None and cardinality < 65500 else np.int32


def get_idx_path(path_prefix: str) -> str:
    return path_prefix + ".idx"


def get_bin_path(path_prefix: str) -> str:
    return path_prefix + ".bin"


def _write_index(idx_path: str, dtype, lengths, modes, document_boundaries) -> None:
    lengths = np.asarray(lengths, dtype=np.int64)
    assert lengths.size == 0 or lengths.max() <= np.iinfo(np.int32).max, "a sequence is longer than int32 allows"
    offsets = np.zeros(lengths.size, dtype=np.int64)
    if lengths.size > 1:
        np.cumsum(lengths[:-1] * DType.size(dtype), out=offsets[1:])
    with open(idx_path, "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<Q", _VERSION))
        f.write(struct.pack("<B", DType.code_from_dtype(dtype)))
        f.write(struct.pack("<Q", lengths.size))
        f.write(struct.pack("<Q", len(document_boundaries)))
        f.write(lengths.astype(np.int32).tobytes(order="C"))
        f.write(offsets.tobytes(order="C"))
        f.write(np.asarray(document_boundaries, dtype=np.int64).tobytes(order="C"))
        if modes is not None:
            f.write(np.asarray(modes, dtype=np.int8).tobytes(order="C"))


class _Index:
    """Zero-copy view of an ``.idx`` file."""

    def __init__(self, idx_path: str, multimodal: bool) -> None:
        with open(idx_path, "rb") as f:
            assert f.read(len(_MAGIC)) == _MAGIC, f"bad header, cannot read: {idx_path}"
            (version,) = struct.unpack("<Q", f.read(8))
            assert version == _VERSION, f"bad version, cannot read: {idx_path}"
            (code,) = struct.unpack("<B", f.read(1))
            (self.sequence_count,) = struct.unpack("<Q", f.read(8))
            (self.document_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self.dtype = DType.dtype_from_code(code)
        self.dtype_size = DType.size(self.dtype)
        self._mmap = np.memmap(idx_path, mode="r", order="C")
        buffer = memoryview(self._mmap)
        self.sequence_lengths = np.frombuffer(buffer, dtype=np.int32, count=self.sequence_count, offset=offset)
        offset += self.sequence_lengths.nbytes
        self.sequence_pointers = np.frombuffer(buffer, dtype=np.int64, count=self.sequence_count, offset=offset)
        offset += self.sequence_pointers.nbytes
        self.document_indices = np.frombuffer(buffer, dtype=np.int64, count=self.document_count, offset=offset)
        offset += self.document_indices.nbytes
        self.sequence_modes = None
        if multimodal:
            self.sequence_modes = np.frombuffer(buffer, dtype=np.int8, count=self.sequence_count, offset=offset)
        assert self.document_count == 0 or self.document_indices[-1] == self.sequence_count

    def __len__(self) -> int:
        return self.sequence_count


class MMapIndexedDataset(torch.utils.data.Dataset):
    """Random access to the sequences of one ``.bin``/``.idx`` pair; picklable by path for dataloader workers."""

    def __init__(self, path_prefix: str, multimodal: bool = False) -> None:
        super().__init__()
        self._open(path_prefix, multimodal)

    def _open(self, path_prefix: str, multimodal: bool) -> None:
        self.path_prefix = path_prefix
        self.multimodal = multimodal
        self.index = _Index(get_idx_path(path_prefix), multimodal)
        self._bin = np.memmap(get_bin_path(path_prefix), mode="r", order="C")
        self._bin_view = memoryview(self._bin)

    def __getstate__(self):
        return self.path_prefix, self.multimodal

    def __setstate__(self, state) -> None:
        self._open(*state)

    def __len__(self) -> int:
        return len(self.index)

    def _read(self, byte_offset: int, count: int) -> np.ndarray:
        return np.frombuffer(self._bin_view, dtype=self.index.dtype, count=int(count), offset=int(byte_offset))

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            tokens = self._read(self.index.sequence_pointers[idx], self.index.sequence_lengths[idx])
            return (tokens, self.index.sequence_modes[idx]) if self.multimodal else tokens
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("slices into the indexed dataset must be contiguous")
            lengths = self.index.sequence_lengths[idx]
            if start >= stop:
                return ([], self.index.sequence_modes[idx]) if self.multimodal else []
            flat = self._read(self.index.sequence_pointers[start], int(lengths.sum()))
            parts = np.split(flat, np.cumsum(lengths)[:-1])
            return (parts, self.index.sequence_modes[idx]) if self.multimodal else parts
        raise TypeError(f"unexpected type received for idx: {type(idx)}")

    def get(self, idx: int, offset: int = 0, length: int | None = None) -> np.ndarray:
        """``length`` tokens of sequence ``idx`` starting ``offset`` tokens in (to its end by default)."""
        if length is None:
            length = self.index.sequence_lengths[idx] - offset
        pointer = self.index.sequence_pointers[idx] + offset * self.index.dtype_size
        tokens = self._read(pointer, length)
        return (tokens, self.index.sequence_modes[idx]) if self.multimodal else tokens

    @property
    def sequence_lengths(self) -> np.ndarray:
        return self.index.sequence_lengths

    @property
    def document_indices(self) -> np.ndarray:
        return self.index.document_indices

    def get_document_indices(self) -> np.ndarray:
        return self.index.document_indices

    def set_document_indices(self, document_indices: np.ndarray) -> None:
        self.index.document_indices = document_indices

    @property
    def sequence_modes(self) -> np.ndarray:
        return self.index.sequence_modes

    @staticmethod
    def exists(path_prefix: str) -> bool:
        return os.path.exists(get_idx_path(path_prefix)) and os.path.exists(get_bin_path(path_prefix))


class MMapIndexedDatasetBuilder:
    """Streams sequences into a ``.bin`` file and writes the ``.idx`` on :meth:`finalize`."""

    def __init__(self, bin_path: str, dtype=np.int32, multimodal: bool = False) -> None:
        self._file = open(bin_path, "wb")
        self.dtype = dtype
        self.multimodal = multimodal
        self.sequence_lengths: list[int] = []
        self.document_indices: list[int] = [0]
        self.sequence_modes: list[int] | None = [] if multimodal else None

    def add_item(self, tensor, mode: int = 0) -> None:
        array = np.asarray(tensor.numpy() if torch.is_tensor(tensor) else tensor, dtype=self.dtype)
        self._file.write(array.tobytes(order="C"))
        self.sequence_lengths.append(array.size)
        if self.multimodal:
            self.sequence_modes.append(mode)

    def add_document(self, tensor, lengths: list[int], modes: list[int] | None = None) -> None:
        array = np.asarray(tensor.numpy() if torch.is_tensor(tensor) else tensor, dtype=self.dtype)
        assert array.size == sum(lengths)
        self._file.write(array.tobytes(order="C"))
        self.sequence_lengths.extend(int(n) for n in lengths)
        self.document_indices.append(len(self.sequence_lengths))
        if self.multimodal:
            self.sequence_modes.extend(modes if modes is not None else [0] * len(lengths))

    def end_document(self) -> None:
        self.document_indices.append(len(self.sequence_lengths))

    def add_index(self, path_prefix: str) -> None:
        """Append another store (same dtype) without re-tokenising: index entries shifted, ``.bin`` bytes copied."""
        other = _Index(get_idx_path(path_prefix), self.multimodal)
        assert np.dtype(other.dtype) == np.dtype(self.dtype), "cannot merge stores of different dtypes"
        base = len(self.sequence_lengths)
        self.sequence_lengths.extend(int(n) for n in other.sequence_lengths)
        self.document_indices.extend(int(base + d) for d in other.document_indices[1:])
        if self.multimodal:
            self.sequence_modes.extend(int(m) for m in other.sequence_modes)
        with open(get_bin_path(path_prefix), "rb") as src:
            shutil.copyfileobj(src, self._file)

    def finalize(self, idx_path: str) -> None:
        self._file.close()
        _write_index(idx_path, self.dtype, self.sequence_lengths, self.sequence_modes, self.document_indices)

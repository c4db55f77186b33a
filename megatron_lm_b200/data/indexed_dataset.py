"""Memory-mapped token datasets in the ``.bin`` / ``.idx`` format.

File format (identical to the reference's, so existing preprocessed corpora load unchanged;
megatron/core/datasets/indexed_dataset.py:45-62,140-300):

``.idx``: magic ``MMIDIDX\\x00\\x00`` | ``<Q`` version = 1 | ``<B`` dtype code | ``<Q`` sequence
count | ``<Q`` document count | int32 sequence lengths | int64 byte offsets of each sequence in
``.bin`` | int64 document boundaries (indices into the sequence arrays, first is 0) | optional
int8 sequence modes (multimodal).  ``.bin``: the raw token arrays back to back.
dtype codes: 1 uint8, 2 int8, 3 int16, 4 int32, 5 int64, 6 float64, 7 float32, 8 uint16.
"""
from __future__ import annotations

import os
import struct
from typing import List, Optional, Tuple, Union

import numpy as np

_MAGIC = b"MMIDIDX\x00\x00"
_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODE_OF = {np.dtype(v): k for k, v in _CODES.items()}


def optimal_dtype(vocab_size: Optional[int]):
    """uint16 when every token id fits, else int32 (reference: indexed_dataset.py:105-118)."""
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def get_idx_path(prefix: str) -> str:
    return prefix + ".idx"


def get_bin_path(prefix: str) -> str:
    return prefix + ".bin"


class _Index:
    def __init__(self, path: str, multimodal: bool = False):
        with open(path, "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError(f"{path} is not an indexed-dataset index (bad magic)")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = np.dtype(_CODES[code])
            (self.sequence_count,) = struct.unpack("<Q", f.read(8))
            (self.document_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._mmap = np.memmap(path, mode="r", order="C")
        buf = memoryview(self._mmap)
        self.sequence_lengths = np.frombuffer(buf, dtype=np.int32, count=self.sequence_count, offset=offset)
        offset += self.sequence_lengths.nbytes
        self.sequence_pointers = np.frombuffer(buf, dtype=np.int64, count=self.sequence_count, offset=offset)
        offset += self.sequence_pointers.nbytes
        self.document_indices = np.frombuffer(buf, dtype=np.int64, count=self.document_count, offset=offset)
        offset += self.document_indices.nbytes
        self.sequence_modes = None
        if multimodal:
            self.sequence_modes = np.frombuffer(buf, dtype=np.int8, count=self.sequence_count, offset=offset)

    def __len__(self):
        return self.sequence_count


class IndexedDataset:
    """Random access to the sequences of a ``.bin``/``.idx`` pair (mmap by default)."""

    def __init__(self, path_prefix: str, multimodal: bool = False, mmap: bool = True, object_storage_config=None):
        self.path_prefix, self.multimodal, self.mmap = path_prefix, multimodal, mmap
        self._remote = None
        from . import object_storage as osu
        if osu.is_object_storage_path(path_prefix):
            # index cached on local disk, tokens read from the store in large cached ranges
            if object_storage_config is None:
                raise ValueError(f"{path_prefix}: an object-storage dataset needs an ObjectStorageConfig "
                                 "(where to cache the index, how large a ranged read is)")
            local_idx = osu.get_index_cache_path(get_idx_path(path_prefix), object_storage_config)
            osu.cache_index_file(get_idx_path(path_prefix), local_idx)
            self.index = _Index(local_idx, multimodal)
            self._remote = osu.ObjectStorageBinReader(get_bin_path(path_prefix), object_storage_config)
            self.mmap = False
            return
        self.index = _Index(get_idx_path(path_prefix), multimodal)
        if mmap:
            self._bin = np.memmap(get_bin_path(path_prefix), mode="r", order="C")
            self._buf = memoryview(self._bin)
        else:
            self._file = open(get_bin_path(path_prefix), "rb")

    def __len__(self) -> int:
        return len(self.index)

    def _read(self, count: int, byte_offset: int) -> np.ndarray:
        if self._remote is not None:
            return self._remote.read(self.index.dtype, count, byte_offset)
        if self.mmap:
            return np.frombuffer(self._buf, dtype=self.index.dtype, count=count, offset=byte_offset)
        self._file.seek(byte_offset)
        out = np.empty(count, dtype=self.index.dtype)
        self._file.readinto(out)
        return out

    def __getitem__(self, idx: Union[int, np.integer, slice]):
        if isinstance(idx, (int, np.integer)):
            seq = self._read(int(self.index.sequence_lengths[idx]), int(self.index.sequence_pointers[idx]))
            return (seq, self.index.sequence_modes[idx]) if self.index.sequence_modes is not None else seq
        start, stop, step = idx.indices(len(self))
        if step != 1:
            raise ValueError("slices into an indexed dataset must be contiguous")
        lengths = self.index.sequence_lengths[start:stop]
        flat = self._read(int(lengths.sum()), int(self.index.sequence_pointers[start]))
        seqs = np.split(flat, np.cumsum(lengths)[:-1])
        if self.index.sequence_modes is not None:
            return seqs, self.index.sequence_modes[start:stop]
        return seqs

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        """``length`` tokens of sequence ``idx`` starting at ``offset``."""
        n = int(self.index.sequence_lengths[idx])
        if length is None:
            length = n - offset
        ptr = int(self.index.sequence_pointers[idx]) + offset * self.index.dtype.itemsize
        return self._read(length, ptr)

    @property
    def sequence_lengths(self) -> np.ndarray:
        return self.index.sequence_lengths

    @property
    def document_indices(self) -> np.ndarray:
        return self.index.document_indices

    @staticmethod
    def exists(path_prefix: str) -> bool:
        from . import object_storage as osu
        if osu.is_object_storage_path(path_prefix):
            return osu.dataset_exists(path_prefix, get_idx_path(path_prefix), get_bin_path(path_prefix))
        return os.path.exists(get_idx_path(path_prefix)) and os.path.exists(get_bin_path(path_prefix))


class IndexedDatasetBuilder:
    """Writes a ``.bin`` and, on ``finalize``, its ``.idx`` (reference: indexed_dataset.py:826)."""

    def __init__(self, bin_path: str, dtype=np.int32, multimodal: bool = False):
        self._f = open(bin_path, "wb")
        self.dtype = np.dtype(dtype)
        self.multimodal = multimodal
        self.sequence_lengths: List[int] = []
        self.document_indices: List[int] = [0]
        self.sequence_modes: Optional[List[int]] = [] if multimodal else None

    def add_item(self, tokens, mode: int = 0) -> None:
        arr = np.asarray(tokens, dtype=self.dtype)
        self._f.write(arr.tobytes(order="C"))
        self.sequence_lengths.append(arr.size)
        if self.multimodal:
            self.sequence_modes.append(mode)

    def add_document(self, tokens, lengths: List[int], modes: Optional[List[int]] = None) -> None:
        arr = np.asarray(tokens, dtype=self.dtype)
        self._f.write(arr.tobytes(order="C"))
        self.sequence_lengths.extend(lengths)
        self.document_indices.append(len(self.sequence_lengths))
        if self.multimodal:
            self.sequence_modes.extend(modes if modes is not None else [0] * len(lengths))

    def end_document(self) -> None:
        self.document_indices.append(len(self.sequence_lengths))

    def add_index(self, path_prefix: str) -> None:
        """Append another dataset (used by the merge tool)."""
        other = _Index(get_idx_path(path_prefix), self.multimodal)
        if other.dtype != self.dtype:
            raise ValueError("cannot merge datasets of different token dtypes")
        base = len(self.sequence_lengths)
        self.sequence_lengths.extend(other.sequence_lengths.tolist())
        self.document_indices.extend((base + other.document_indices[1:]).tolist())
        if self.multimodal:
            self.sequence_modes.extend(other.sequence_modes.tolist())
        with open(get_bin_path(path_prefix), "rb") as f:
            while True:
                chunk = f.read(1 << 24)
                if not chunk:
                    break
                self._f.write(chunk)

    def finalize(self, idx_path: str) -> None:
        self._f.close()
        lengths = np.asarray(self.sequence_lengths, dtype=np.int32)
        pointers = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        with open(idx_path, "wb") as f:
            f.write(_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", _CODE_OF[self.dtype]))
            f.write(struct.pack("<Q", len(lengths)))
            f.write(struct.pack("<Q", len(self.document_indices)))
            f.write(lengths.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self.document_indices, dtype=np.int64).tobytes(order="C"))
            if self.multimodal:
                f.write(np.asarray(self.sequence_modes, dtype=np.int8).tobytes(order="C"))

"""Memory-mapped indexed token dataset (`<prefix>.bin` + `<prefix>.idx`), reader and builder.

File format of the Megatron `mmap` implementation (reference:
eth/runtime/megatron/data/indexed_dataset.py:335-570): the index starts with the magic
`MMIDIDX\\x00\\x00`, a uint64 version (1), a uint8 dtype code, uint64 sequence and document counts,
then int32 sizes, int64 byte pointers and int64 document boundaries; the data file is the raw
token stream.
"""
from __future__ import annotations

import os
import struct
from typing import List, Sequence

import numpy as np

MAGIC = b"MMIDIDX\x00\x00"
DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}


def dtype_code(dtype) -> int:
    for k, v in DTYPES.items():
        if np.dtype(v) == np.dtype(dtype):
            return k
    raise ValueError(f"unsupported dtype {dtype}")


def index_file_path(prefix: str) -> str:
    return prefix + ".idx"


def data_file_path(prefix: str) -> str:
    return prefix + ".bin"


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file: str, dtype=np.int32):
        self._data = open(out_file, "wb")
        self._dtype = np.dtype(dtype)
        self._sizes: List[int] = []
        self._doc_idx: List[int] = [0]

    def add_item(self, tokens: Sequence[int]) -> None:
        arr = np.asarray(tokens, dtype=self._dtype)
        self._data.write(arr.tobytes(order="C"))
        self._sizes.append(arr.size)

    def end_document(self) -> None:
        self._doc_idx.append(len(self._sizes))

    def finalize(self, index_file: str) -> None:
        self._data.close()
        sizes = np.asarray(self._sizes, dtype=np.int32)
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * self._dtype.itemsize, out=pointers[1:])
        with open(index_file, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", dtype_code(self._dtype)))
            f.write(struct.pack("<Q", len(sizes)))
            f.write(struct.pack("<Q", len(self._doc_idx)))
            f.write(sizes.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self._doc_idx, dtype=np.int64).tobytes(order="C"))


class MMapIndexedDataset:
    def __init__(self, prefix: str):
        self.prefix = prefix
        with open(index_file_path(prefix), "rb") as f:
            if f.read(9) != MAGIC:
                raise ValueError(f"{index_file_path(prefix)} is not an mmap index file")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = np.dtype(DTYPES[code])
            (n,) = struct.unpack("<Q", f.read(8))
            (ndoc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._index = np.memmap(index_file_path(prefix), mode="r", order="C")
        self.sizes = np.frombuffer(self._index, dtype=np.int32, count=n, offset=offset)
        self._pointers = np.frombuffer(self._index, dtype=np.int64, count=n, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(self._index, dtype=np.int64, count=ndoc,
                                     offset=offset + self.sizes.nbytes + self._pointers.nbytes)
        self._data = np.memmap(data_file_path(prefix), mode="r", order="C")

    def __len__(self) -> int:
        return len(self.sizes)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return [self[i] for i in range(*idx.indices(len(self)))]
        return np.frombuffer(self._data, dtype=self.dtype, count=int(self.sizes[idx]), offset=int(self._pointers[idx]))

    def get(self, idx: int, offset: int = 0, length=None):
        size = int(self.sizes[idx])
        length = size - offset if length is None else length
        return np.frombuffer(self._data, dtype=self.dtype, count=length,
                             offset=int(self._pointers[idx]) + offset * self.dtype.itemsize)

    @staticmethod
    def exists(prefix: str) -> bool:
        return os.path.exists(index_file_path(prefix)) and os.path.exists(data_file_path(prefix))


def make_dataset(prefix: str, impl: str = "mmap"):
    if impl not in ("mmap", "infer"):
        raise ValueError(f"data implementation {impl!r} is not available; use mmap")
    if not MMapIndexedDataset.exists(prefix):
        raise FileNotFoundError(f"dataset {prefix}.bin/.idx does not exist")
    return MMapIndexedDataset(prefix)

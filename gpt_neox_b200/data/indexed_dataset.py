"""Memory-mapped token datasets (``<prefix>.bin`` + ``<prefix>.idx``).

On-disk format (byte compatible with ``megatron/data/indexed_dataset.py:340-595``, so corpora
tokenised for GPT-NeoX load unchanged):

``.idx``  ``b"MMIDIDX\\x00\\x00"`` | ``<Q`` version = 1 | ``<B`` dtype code | ``<Q`` number of sequences |
          ``<Q`` number of document boundaries | int32 sizes[n] | int64 byte pointers[n] | int64 doc_idx[d]
``.bin``  the token arrays back to back.

dtype codes: 1 uint8, 2 int8, 3 int16, 4 int32, 5 int64, 6 float32, 7 float64, 8 uint16.
The legacy ``TNTIDX`` format is read too (``IndexedDataset``).
"""
from __future__ import annotations

import os
import struct

import numpy as np
import torch

DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
_MAGIC = b"MMIDIDX\x00\x00"
_LEGACY_MAGIC = b"TNTIDX\x00\x00"


def dtype_code(dtype) -> int:
    for k, v in DTYPES.items():
        if v == dtype:
            return k
    raise ValueError(dtype)


def best_fitting_dtype(vocab_size=None):
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def index_file_path(prefix):
    return prefix + ".idx"


def data_file_path(prefix):
    return prefix + ".bin"


def infer_dataset_impl(path):
    if not MMapIndexedDataset.exists(path):
        print(f"Dataset does not exist: {path}")
        return None
    with open(index_file_path(path), "rb") as fh:
        magic = fh.read(9)
    if magic[:8] == _LEGACY_MAGIC[:8]:
        return "cached"
    if magic == _MAGIC:
        return "mmap"
    return None


class MMapIndexedDataset(torch.utils.data.Dataset):
    def __init__(self, path, skip_warmup=True):
        super().__init__()
        self._path = path
        with open(index_file_path(path), "rb") as fh:
            assert fh.read(9) == _MAGIC, "Index file doesn't match expected format. Make sure that --dataset-impl is configured properly."
            (version,) = struct.unpack("<Q", fh.read(8))
            assert version == 1
            (code,) = struct.unpack("<B", fh.read(1))
            self._dtype = DTYPES[code]
            (self._len,) = struct.unpack("<Q", fh.read(8))
            (self._doc_count,) = struct.unpack("<Q", fh.read(8))
            offset = fh.tell()
        if not skip_warmup:
            with open(index_file_path(path), "rb") as fh:
                while fh.read(100 * 1024 * 1024):
                    pass
        self._idx_mm = np.memmap(index_file_path(path), mode="r", order="C")
        buf = memoryview(self._idx_mm)
        self._sizes = np.frombuffer(buf, dtype=np.int32, count=self._len, offset=offset)
        self._pointers = np.frombuffer(buf, dtype=np.int64, count=self._len, offset=offset + self._sizes.nbytes)
        self._doc_idx = np.frombuffer(buf, dtype=np.int64, count=self._doc_count,
                                      offset=offset + self._sizes.nbytes + self._pointers.nbytes)
        self._bin_mm = np.memmap(data_file_path(path), mode="r", order="C")
        self._bin = memoryview(self._bin_mm)

    def __getstate__(self):
        return self._path

    def __setstate__(self, state):
        self.__init__(state)

    def __len__(self):
        return self._len

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            return np.frombuffer(self._bin, dtype=self._dtype, count=int(self._sizes[idx]),
                                 offset=int(self._pointers[idx]))
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("Slices into indexed_dataset must be contiguous")
            sizes = self._sizes[idx]
            total = int(sum(sizes))
            arr = np.frombuffer(self._bin, dtype=self._dtype, count=total, offset=int(self._pointers[start]))
            return np.split(arr, np.cumsum(sizes)[:-1])
        raise TypeError(idx)

    def get(self, idx, offset=0, length=None):
        """Tokens ``[offset, offset+length)`` of sequence ``idx`` without touching the rest."""
        size = int(self._sizes[idx])
        if length is None:
            length = size - offset
        ptr = int(self._pointers[idx]) + offset * np.dtype(self._dtype).itemsize
        return np.frombuffer(self._bin, dtype=self._dtype, count=length, offset=ptr)

    @property
    def sizes(self):
        return self._sizes

    @property
    def doc_idx(self):
        return self._doc_idx

    def get_doc_idx(self):
        return self._doc_idx

    def set_doc_idx(self, doc_idx):
        self._doc_idx = doc_idx

    @property
    def dtype(self):
        return self._dtype

    @property
    def supports_prefetch(self):
        return False

    @staticmethod
    def exists(path):
        return os.path.exists(index_file_path(path)) and os.path.exists(data_file_path(path))


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file, dtype=np.int64):
        self._data_file = open(out_file, "wb")
        self._dtype = dtype
        self._sizes = []
        self._doc_idx = [0]

    @property
    def dtype(self):
        return self._dtype

    def add_item(self, np_array):
        arr = np.asarray(np_array, dtype=self._dtype)
        self._data_file.write(arr.tobytes(order="C"))
        self._sizes.append(arr.size)

    def add_items(self, arr_list):
        for a in arr_list:
            self.add_item(a)

    def end_document(self):
        self._doc_idx.append(len(self._sizes))

    def merge_file_(self, another_file):
        other = MMapIndexedDataset(another_file)
        assert other.dtype == self._dtype
        base = len(self._sizes)
        self._sizes.extend(int(s) for s in other.sizes)
        self._doc_idx.extend(int(d) + base for d in other.doc_idx[1:])
        with open(data_file_path(another_file), "rb") as fh:
            while True:
                chunk = fh.read(1 << 24)
                if not chunk:
                    break
                self._data_file.write(chunk)

    def finalize(self, index_file):
        self._data_file.close()
        sizes = np.array(self._sizes, dtype=np.int64)
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1], out=pointers[1:])
        pointers *= np.dtype(self._dtype).itemsize
        with open(index_file, "wb") as fh:
            fh.write(_MAGIC)
            fh.write(struct.pack("<Q", 1))
            fh.write(struct.pack("<B", dtype_code(self._dtype)))
            fh.write(struct.pack("<Q", len(sizes)))
            fh.write(struct.pack("<Q", len(self._doc_idx)))
            fh.write(sizes.astype(np.int32).tobytes(order="C"))
            fh.write(pointers.tobytes(order="C"))
            fh.write(np.array(self._doc_idx, dtype=np.int64).tobytes(order="C"))


class IndexedDataset(torch.utils.data.Dataset):
    """Reader of the legacy ``TNTIDX`` format (whole-file reads, optional caching)."""

    def __init__(self, path, cached=False):
        super().__init__()
        self.path = path
        with open(index_file_path(path), "rb") as fh:
            assert fh.read(8) == _LEGACY_MAGIC[:8], "Index file doesn't match expected format."
            assert struct.unpack("<Q", fh.read(8)) == (1,)
            code, self.element_size = struct.unpack("<QQ", fh.read(16))
            self.dtype = DTYPES[code]
            self._len, self.s = struct.unpack("<QQ", fh.read(16))
            (self.doc_count,) = struct.unpack("<Q", fh.read(8))
            self.dim_offsets = np.fromfile(fh, dtype=np.int64, count=self._len + 1)
            self.data_offsets = np.fromfile(fh, dtype=np.int64, count=self._len + 1)
            self.sizes = np.fromfile(fh, dtype=np.int64, count=self.s)
            self.doc_idx = np.fromfile(fh, dtype=np.int64, count=self.doc_count)
        self._data = np.memmap(data_file_path(path), mode="r", dtype=self.dtype)
        self._cache = {} if cached else None

    def __len__(self):
        return self._len

    def __getitem__(self, i):
        if self._cache is not None and i in self._cache:
            return self._cache[i]
        a = np.array(self._data[self.data_offsets[i]:self.data_offsets[i + 1]])
        if self._cache is not None:
            self._cache[i] = a
        return a

    @staticmethod
    def exists(path):
        return os.path.exists(index_file_path(path)) and os.path.exists(data_file_path(path))


def make_dataset(path, impl, skip_warmup=True):
    if not MMapIndexedDataset.exists(path):
        print(f"Dataset does not exist: {path}")
        print("Path should be a basename that both .idx and .bin can be appended to get full filenames.")
        return None
    if impl == "infer":
        impl = infer_dataset_impl(path)
    if impl == "cached":
        return IndexedDataset(path, cached=True)
    if impl == "mmap":
        return MMapIndexedDataset(path, skip_warmup)
    print(f"Unknown dataset implementation: {impl}")
    return None


def make_builder(out_file, impl, vocab_size=None):
    return MMapIndexedDatasetBuilder(out_file, dtype=best_fitting_dtype(vocab_size))

"""Read single-file and sharded safetensors checkpoints into numpy arrays.

Mirrors python/mojolearn/models/safetensors.py of the reference (:1-159): F32, I32 and I64 keep their stored bytes;
F16 and BF16 widen EXACTLY to float32 (a shift for BF16, the bit construction below for F16), or, with
`bf16="bits"`, a BF16 matrix stays as its uint16 bits inside a `lowbit.BF16Weight`; every other storage type is
refused by name. A checkpoint is a `model.safetensors`, an explicit `.safetensors` path, or a directory with
`model.safetensors.index.json` and its shards. Host-side byte work only: nothing here touches a GPU.

The file format: an 8-byte little-endian header length, a JSON header mapping each tensor name to its dtype, shape
and [begin, end) byte offsets into the data section that follows the header.
"""
import json
import os
import struct

import numpy as np

from .. import lowbit

DTYPES = {"F32": ("<f4", 4), "F16": ("<u2", 2), "BF16": ("<u2", 2), "I32": ("<i4", 4), "I64": ("<i8", 8)}
INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


def widen_f16(bits):
    """float16 bit patterns (uint16, any shape) to float32 by bit construction: a normal value keeps its mantissa
    shifted up by 13 with the exponent rebiased by 112, a subnormal is renormalised into a normal float32, zero keeps
    its sign, infinities and NaNs keep sign and payload. Exact."""
    h = np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32)
    sign, exp, man = (h & 0x8000) << 16, (h >> 10) & 0x1F, h & 0x3FF
    out = np.empty(h.shape, dtype=np.uint32)
    normal = (exp > 0) & (exp < 31)
    out[normal] = sign[normal] | ((exp[normal] + 112) << 23) | (man[normal] << 13)
    special = exp == 31
    out[special] = sign[special] | 0x7F800000 | (man[special] << 13)
    zero = (exp == 0) & (man == 0)
    out[zero] = sign[zero]
    sub = (exp == 0) & (man != 0)
    if sub.any():
        m = man[sub]
        shift = np.zeros(m.shape, dtype=np.uint32)
        for _ in range(10):  # bring the leading one of the 10-bit mantissa up to bit 10
            small = (m & 0x400) == 0
            m = np.where(small, m << 1, m)
            shift = shift + small.astype(np.uint32)
        out[sub] = sign[sub] | ((113 - shift) << 23) | ((m & 0x3FF) << 13)
    return out.view(np.float32)


class TensorInfo(object):
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, tuple(shape), begin, end, file

    @property
    def nbytes(self):
        return self.end - self.begin

    @property
    def size(self):
        return int(np.prod(self.shape)) if self.shape else 1


class SafetensorsFile(object):
    """One `.safetensors` file: `names()`, `info(name)`, `read(name)`; a context manager that releases the map."""

    def __init__(self, path):
        self.path = str(path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise ValueError("%s: not a safetensors file (shorter than its length word)" % self.path)
            (hlen,) = struct.unpack("<Q", head)
            if hlen <= 0 or hlen > os.path.getsize(self.path) - 8:
                raise ValueError("%s: header length %d does not fit the file" % (self.path, hlen))
            header = json.loads(f.read(hlen).decode("utf-8"))
        self._data0 = 8 + hlen
        self._map = None
        self._info = {}
        data_bytes = os.path.getsize(self.path) - self._data0
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            begin, end = entry["data_offsets"]
            info = TensorInfo(name, entry["dtype"], entry["shape"], int(begin), int(end), self.path)
            if info.dtype in DTYPES and info.nbytes != info.size * DTYPES[info.dtype][1]:
                raise ValueError("%s: tensor %r holds %d bytes, its shape and dtype say %d" %
                                 (self.path, name, info.nbytes, info.size * DTYPES[info.dtype][1]))
            if begin < 0 or end > data_bytes or begin > end:
                raise ValueError("%s: tensor %r lies outside the data section" % (self.path, name))
            self._info[name] = info

    def names(self):
        return sorted(self._info)

    def info(self, name):
        if name not in self._info:
            raise KeyError("%s holds no tensor %r" % (self.path, name))
        return self._info[name]

    def __contains__(self, name):
        return name in self._info

    def read(self, name, *, bf16="widen"):
        """The tensor as an owned array; `bf16` = "widen" (float32) or "bits" (uint16 bits, a matrix as a BF16Weight)."""
        if bf16 not in ("widen", "bits"):
            raise ValueError("bf16 must be 'widen' or 'bits'")
        info = self.info(name)
        if info.dtype not in DTYPES:
            raise TypeError("%s: tensor %r is stored as %s, which is not read (F32, F16, BF16, I32 and I64 are)" %
                            (self.path, name, info.dtype))
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="r")
        raw = np.array(self._map[self._data0 + info.begin:self._data0 + info.end])  # an owned copy of the bytes
        arr = raw.view(DTYPES[info.dtype][0]).reshape(info.shape)
        if info.dtype == "F16":
            return widen_f16(arr)
        if info.dtype == "BF16":
            if bf16 == "bits":
                return lowbit.BF16Weight(arr) if arr.ndim == 2 else arr
            return (arr.astype(np.uint32) << 16).view(np.float32)
        return arr

    def close(self):
        self._map = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


class Checkpoint(object):
    """A single `model.safetensors`, an explicit `.safetensors` path, or a directory holding
    `model.safetensors.index.json` and its shards (opened on first use, closed by `close()`)."""

    def __init__(self, files, weight_map, root):
        self._files, self._weight_map, self.root = files, weight_map, root

    @classmethod
    def open(cls, path):
        path = str(path)
        if os.path.isfile(path):
            f = SafetensorsFile(path)
            return cls({path: f}, {n: path for n in f.names()}, os.path.dirname(path))
        index = os.path.join(path, INDEX_NAME)
        single = os.path.join(path, SINGLE_NAME)
        if os.path.isfile(index):
            weight_map = json.load(open(index))["weight_map"]
            return cls({}, {n: os.path.join(path, rel) for n, rel in weight_map.items()}, path)
        if os.path.isfile(single):
            return cls.open(single)
        raise FileNotFoundError("%s holds neither %s nor %s" % (path, SINGLE_NAME, INDEX_NAME))

    def _file(self, path):
        if path not in self._files:
            self._files[path] = SafetensorsFile(path)
        return self._files[path]

    def names(self):
        return sorted(self._weight_map)

    def __contains__(self, name):
        return name in self._weight_map

    def info(self, name):
        if name not in self._weight_map:
            raise KeyError("the checkpoint holds no tensor %r" % name)
        return self._file(self._weight_map[name]).info(name)

    def read(self, name, *, bf16="widen"):
        if name not in self._weight_map:
            raise KeyError("the checkpoint holds no tensor %r" % name)
        return self._file(self._weight_map[name]).read(name, bf16=bf16)

    def close(self):
        for f in self._files.values():
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def write_file(path, tensors):
    """Write float32 / int32 / int64 / uint16-as-BF16 arrays as one safetensors file (used by tests and to export a
    model): the inverse of SafetensorsFile for the storage types it keeps byte for byte."""
    names = {np.dtype("<f4"): "F32", np.dtype("<i4"): "I32", np.dtype("<i8"): "I64", np.dtype("<u2"): "BF16"}
    header, blobs, at = {}, [], 0
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        if a.dtype not in names:
            raise TypeError("tensor %r has dtype %s, which is not written" % (name, a.dtype))
        raw = a.tobytes()
        header[name] = {"dtype": names[a.dtype], "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)

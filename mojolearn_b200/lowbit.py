"""Low-bit WEIGHT STORAGE: bf16 bits or int8 codes with one power-of-two
exponent per row, materialised exactly to float32 by whoever computes with them.

Mirrors python/mojolearn/lowbit.py of the reference (:38-178): `pack` /
`unpack` walk a weights dict and convert every 2-D tensor, `pack_one` /
`materialize_one` convert one, `format_of` / `is_packed` are the predicates,
`widen_bf16` takes bits of any rank. The conversions run on the GPU through
mojolearn_b200.linalg; there is no host fallback.
"""
import numpy as np

from . import linalg

FORMATS = ("float32", "bfloat16", "int8")


class BF16Weight(object):
    """A 2-D weight held as bfloat16 bit patterns (uint16)."""
    format = "bfloat16"

    def __init__(self, bits):
        bits = np.ascontiguousarray(bits)
        if bits.dtype != np.uint16 or bits.ndim != 2:
            raise TypeError("BF16Weight holds a 2-D uint16 array of bfloat16 bits")
        self.bits = bits

    @property
    def shape(self):
        return self.bits.shape


class Int8Weight(object):
    """A 2-D weight held as int8 codes and one int32 exponent per row: row = codes * 2**exponent."""
    format = "int8"

    def __init__(self, codes, exponents):
        codes = np.ascontiguousarray(codes)
        exponents = np.ascontiguousarray(exponents)
        if codes.dtype != np.int8 or codes.ndim != 2:
            raise TypeError("Int8Weight codes are a 2-D int8 array")
        if exponents.dtype != np.int32 or exponents.shape != (codes.shape[0],):
            raise TypeError("Int8Weight exponents are int32, one per row")
        self.codes, self.exponents = codes, exponents

    @property
    def shape(self):
        return self.codes.shape


def is_packed(x):
    return isinstance(x, (BF16Weight, Int8Weight))


def pack_one(x, fmt):
    """One 2-D float32 tensor in storage format `fmt`."""
    if fmt not in FORMATS:
        raise ValueError("unknown format %r (one of %s)" % (fmt, ", ".join(FORMATS)))
    a = np.asarray(x)
    if a.ndim != 2:
        raise ValueError("a tensor must be 2-D to pack, got %d-D" % a.ndim)
    if a.dtype != np.float32:
        raise TypeError("pack_one takes float32, got %s" % a.dtype)
    if fmt == "float32":
        return np.array(a, copy=True)
    if fmt == "bfloat16":
        return BF16Weight(linalg.to_bf16(a))
    return Int8Weight(*linalg.quantize_int8(a))


def materialize_one(x):
    """The exact float32 tensor a stored weight stands for."""
    if isinstance(x, BF16Weight):
        return linalg.from_bf16(x.bits)
    if isinstance(x, Int8Weight):
        return linalg.dequantize_int8(x.codes, x.exponents)
    return np.asarray(x)


def widen_bf16(bits):
    """bfloat16 bits of ANY rank to float32 (norm weights, embedding tables)."""
    return linalg.from_bf16(np.asarray(bits))


def _values(weights):
    return list(weights.values()) if isinstance(weights, dict) else list(weights)


def format_of(weights):
    """The storage format of a weights collection; a mix of two low-bit formats is refused."""
    seen = set()
    for w in _values(weights):
        if is_packed(w):
            seen.add(w.format)
    if len(seen) > 1:
        raise ValueError("weights mix %s: store a model one way" % " and ".join(sorted(seen)))
    return seen.pop() if seen else "float32"


def pack(weights, fmt):
    """Every 2-D tensor of `weights` (a dict) packed; other ranks stay float32."""
    out = {}
    for name, w in weights.items():
        a = np.asarray(w)
        out[name] = pack_one(a, fmt) if (a.ndim == 2 and not is_packed(w)) else w
    return out


def unpack(weights):
    return {name: materialize_one(w) for name, w in weights.items()}

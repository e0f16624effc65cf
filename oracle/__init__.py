"""CPU oracle for the identical-mode matrix product (TEST INFRASTRUCTURE).

This package is the checker, not the product: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it. It wraps
liboracle.so (oracle.c, cpu_rows.c, decoder_oracle.c) with numpy arrays.

Every function restates a piece of the reference's host algorithm; the C
sources cite the reference file and lines each one follows. The restatement is
pinned by the reference's committed golden hashes (tests/test_oracle_golden.py).
"""
import ctypes
import hashlib
import os

import numpy as np

from . import build as _build

OP_NN, OP_NT, OP_TN = 0, 1, 2

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path):
            path = _build.build()
        _LIB = ctypes.CDLL(path)
        i64, f32p = ctypes.c_int64, ctypes.c_void_p
        _LIB.oracle_leaf_size.restype = i64
        _LIB.oracle_leaf_size.argtypes = [i64]
        _LIB.oracle_leaf_count.restype = i64
        _LIB.oracle_leaf_count.argtypes = [i64]
        _LIB.oracle_leaf_count_at.restype = i64
        _LIB.oracle_leaf_count_at.argtypes = [i64, i64]
        for name in ("oracle_fold_level_width", "oracle_fold_level_base", "oracle_fold_node_addr"):
            getattr(_LIB, name).restype = i64
        _LIB.oracle_fold_level_width.argtypes = [i64, i64]
        _LIB.oracle_fold_level_base.argtypes = [i64, i64]
        _LIB.oracle_fold_node_addr.argtypes = [i64, i64, i64]
        _LIB.oracle_fold_level_count.restype = i64
        _LIB.oracle_fold_level_count.argtypes = [i64]
        _LIB.oracle_fold_node_total.restype = i64
        _LIB.oracle_fold_node_total.argtypes = [i64]
        _LIB.oracle_fold_node_is_carry.restype = ctypes.c_int
        _LIB.oracle_fold_node_is_carry.argtypes = [i64, i64, i64]
        for name in ("oracle_fold_balanced_tree", "oracle_fold_serial", "oracle_fold_padded_pow2", "oracle_fold_stride"):
            getattr(_LIB, name).restype = ctypes.c_float
            getattr(_LIB, name).argtypes = [f32p, i64]
        _LIB.oracle_chain_variant.restype = ctypes.c_float
        _LIB.oracle_chain_variant.argtypes = [f32p, f32p, i64, ctypes.c_int]
        _LIB.oracle_ftz.restype = ctypes.c_float
        _LIB.oracle_ftz.argtypes = [ctypes.c_float]
        _LIB.oracle_gemm.argtypes = [f32p, f32p, f32p, ctypes.c_int, i64, i64, i64]
        _LIB.oracle_gemm_serial.argtypes = [f32p, f32p, f32p, ctypes.c_int, i64, i64, i64]
        _LIB.oracle_gemm_at_leaf.argtypes = [f32p, f32p, f32p, ctypes.c_int, i64, i64, i64, i64]
        _LIB.rows_gemm.argtypes = [f32p, f32p, f32p, ctypes.c_int, i64, i64, i64, ctypes.c_int]
        _LIB.oracle_nan_canon.argtypes = [f32p, i64]
        _LIB.oracle_from_bf16.argtypes = [f32p, f32p, i64]
        _LIB.oracle_to_bf16.argtypes = [f32p, f32p, i64]
        _LIB.oracle_quantize_int8.argtypes = [f32p, f32p, f32p, i64, i64]
        _LIB.oracle_dequantize_int8.argtypes = [f32p, f32p, f32p, i64, i64]
        _LIB.oracle_dequantize_int8_scaled.argtypes = [f32p, f32p, f32p, i64, i64]
        _LIB.oracle_gemm_int8.argtypes = [f32p, f32p, f32p, f32p, f32p, i64, i64, i64]
        _LIB.oracle_fnv1a64.restype = ctypes.c_uint64
        _LIB.oracle_fnv1a64.argtypes = [f32p, i64]
        _LIB.oracle_card_fill.argtypes = [f32p, i64, i64]
    return _LIB


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    a = np.ascontiguousarray(a)
    if a.dtype != np.float32:
        raise TypeError("the oracle takes float32 operands, got %s" % a.dtype)
    return a


def leaf_size(k):
    return int(lib().oracle_leaf_size(int(k)))


def leaf_count(k):
    return int(lib().oracle_leaf_count(int(k)))


def ftz(x):
    return np.float32(lib().oracle_ftz(ctypes.c_float(float(x))))


def _dims(a, b, op):
    if op == OP_NN:
        (m, k), (k2, n) = a.shape, b.shape
    elif op == OP_NT:
        (m, k), (n, k2) = a.shape, b.shape
    elif op == OP_TN:
        (k, m), (k2, n) = a.shape, b.shape
    else:
        raise ValueError("unknown op %r" % (op,))
    if k != k2:
        raise ValueError("contraction extents disagree: %d and %d" % (k, k2))
    return m, n, k


def gemm(a, b, op=OP_NN, leaf=None, serial=False):
    """The normative product (scalar, single thread). `leaf` forces an
    adversarial leaf size; `serial` is the whole-k diagnostic chain."""
    a, b = _f32(a), _f32(b)
    m, n, k = _dims(a, b, op)
    c = np.empty((m, n), dtype=np.float32)
    if serial:
        rc = lib().oracle_gemm_serial(_ptr(c), _ptr(a), _ptr(b), op, m, n, k)
    elif leaf is not None:
        rc = lib().oracle_gemm_at_leaf(_ptr(c), _ptr(a), _ptr(b), op, m, n, k, int(leaf))
    else:
        rc = lib().oracle_gemm(_ptr(c), _ptr(a), _ptr(b), op, m, n, k)
    if rc != 0:
        raise ValueError("oracle refused the product (status %d)" % rc)
    return c


def gemm_rows(a, b, op=OP_NN, threads=None):
    """The same bits at CPU speed (AVX2, threaded): the timed CPU baseline."""
    a, b = _f32(a), _f32(b)
    m, n, k = _dims(a, b, op)
    c = np.empty((m, n), dtype=np.float32)
    if threads is None:
        threads = os.cpu_count() or 1
    rc = lib().rows_gemm(_ptr(c), _ptr(a), _ptr(b), op, m, n, k, int(threads))
    if rc == 2:
        raise RuntimeError("the CPU baseline needs AVX2 and FMA")
    if rc != 0:
        raise ValueError("cpu_rows refused the product (status %d)" % rc)
    return c


def nan_canon(c):
    c = np.array(_f32(c), copy=True)
    lib().oracle_nan_canon(_ptr(c), c.size)
    return c


def fold(partials, kind="tree"):
    p = _f32(np.asarray(partials, dtype=np.float32))
    fn = {"tree": lib().oracle_fold_balanced_tree, "serial": lib().oracle_fold_serial,
          "padded": lib().oracle_fold_padded_pow2, "stride": lib().oracle_fold_stride}[kind]
    return np.float32(fn(_ptr(p), p.size))


def chain(a, b, mode=0):
    a, b = _f32(a).ravel(), _f32(b).ravel()
    return np.float32(lib().oracle_chain_variant(_ptr(a), _ptr(b), a.size, int(mode)))


def from_bf16(bits):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().oracle_from_bf16(_ptr(out), _ptr(bits), bits.size)
    return out


def to_bf16(x):
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_to_bf16(_ptr(out), _ptr(x), x.size)
    return out


def quantize_int8(x):
    x = _f32(x)
    rows, cols = x.shape
    q = np.empty((rows, cols), dtype=np.int8)
    e = np.empty((rows,), dtype=np.int32)
    lib().oracle_quantize_int8(_ptr(q), _ptr(e), _ptr(x), rows, cols)
    return q, e


def dequantize_int8(q, e):
    q = np.ascontiguousarray(q, dtype=np.int8)
    e = np.ascontiguousarray(e, dtype=np.int32)
    rows, cols = q.shape
    y = np.empty((rows, cols), dtype=np.float32)
    lib().oracle_dequantize_int8(_ptr(y), _ptr(q), _ptr(e), rows, cols)
    return y


def dequantize_int8_scaled(q, scale):
    q = np.ascontiguousarray(q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    rows, cols = q.shape
    y = np.empty((rows, cols), dtype=np.float32)
    lib().oracle_dequantize_int8_scaled(_ptr(y), _ptr(q), _ptr(scale), rows, cols)
    return y


def gemm_int8(qa, ea, qb, eb):
    qa = np.ascontiguousarray(qa, dtype=np.int8)
    qb = np.ascontiguousarray(qb, dtype=np.int8)
    ea = np.ascontiguousarray(ea, dtype=np.int32)
    eb = np.ascontiguousarray(eb, dtype=np.int32)
    (m, k), (n, k2) = qa.shape, qb.shape
    if k != k2:
        raise ValueError("contraction extents disagree")
    c = np.empty((m, n), dtype=np.float32)
    rc = lib().oracle_gemm_int8(_ptr(c), _ptr(qa), _ptr(ea), _ptr(qb), _ptr(eb), m, n, k)
    if rc != 0:
        raise ValueError("oracle refused the int8 product")
    return c


def fnv1a64(array):
    a = np.ascontiguousarray(array)
    return int(lib().oracle_fnv1a64(_ptr(a), a.nbytes))


def card_fill(count, salt):
    out = np.empty((int(count),), dtype=np.float32)
    lib().oracle_card_fill(_ptr(out), out.size, int(salt))
    return out


def sha16(*arrays):
    """The verify table's cell hash: sha256 over dtype, shape and bytes of each
    array, first 16 hex digits (tools/identity_break.py:1355-1371)."""
    m = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(np.asarray(a))
        m.update(str(a.dtype).encode())
        m.update(str(a.shape).encode())
        m.update(a.tobytes())
    return m.hexdigest()[:16]


def train_hash(parts):
    """Hash of a lane's parts dict spelled `key=value`, sorted, joined by `|`
    (tools/identity_break.py:1374-1380)."""
    text = "|".join("%s=%s" % (k, v) for k, v in sorted(parts.items()))
    return sha16(np.frombuffer(text.encode(), dtype=np.uint8))

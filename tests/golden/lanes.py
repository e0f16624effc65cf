"""The verify-table lanes on the matrix-product path, restated against a small
`impl` interface so the same lane runs on the CPU oracle and on the CUDA
package. Each returns the lane's `parts` dict (name -> 16-hex-digit hash);
`oracle.train_hash(parts)` is then the table's `train` cell.

They follow tools/identity_break.py of the reference: gemm-pinned :2984-2994,
gemm-transposed :5880-5891, gemm-bf16 :3825-3836, gemm-int8 :3839-3849,
lowbit-conversions :4159-4300 (data parts; the `flags` vector is a record of
API predicates and agreements that hold by construction here).

`impl` provides: matmul(a, b, transpose_a=False, transpose_b=False),
matmul_bf16(a, b_bits, transpose_b=False) with a float32 or uint16 bits,
matmul_int8((qa, ea), (qb, eb)), to_bf16, from_bf16, quantize_int8,
dequantize_int8, and for gemm-int15 (:3852-3879) quantize_int15, dequantize_int15,
matmul_int15 and INT15_MAX_K.
"""
import hashlib

import numpy as np


def sha16(*arrays):
    m = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(np.asarray(a))
        m.update(str(a.dtype).encode())
        m.update(str(a.shape).encode())
        m.update(a.tobytes())
    return m.hexdigest()[:16]


def gemm_pinned(impl, X):
    a = X[:256].T.copy()
    if X.size >= 256 * 4096:
        wide = np.ascontiguousarray(X[:4096, :].reshape(-1)[: 256 * 4096].reshape(256, 4096))
    else:
        wide = X[:256, :]
    c1 = impl.matmul(a.astype(np.float32), X[:256].astype(np.float32))
    if wide.shape[1] == 4096:
        c2 = impl.matmul(wide.astype(np.float32), np.ascontiguousarray(wide[:128].T).astype(np.float32))
    else:
        c2 = c1
    return dict(small=sha16(c1), wide=sha16(c2))


def gemm_transposed(impl, X):
    a = np.ascontiguousarray(X[:256]).astype(np.float32)
    b = np.ascontiguousarray(X[256:384]).astype(np.float32)
    nt = impl.matmul(a, b, transpose_b=True)
    at = np.ascontiguousarray(X[:256].T).astype(np.float32)
    c = np.ascontiguousarray(X[384:384 + at.shape[0]]).astype(np.float32)
    tn = impl.matmul(at, c, transpose_a=True)
    return dict(nt=sha16(nt), tn=sha16(tn))


def gemm_bf16(impl, X):
    a = np.ascontiguousarray(X[:256]).astype(np.float32)
    b = np.ascontiguousarray(X[256:256 + 128]).astype(np.float32)
    bb = np.asarray(impl.to_bf16(b))
    c1 = impl.matmul_bf16(a, bb, transpose_b=True)
    c2 = impl.matmul_bf16(np.asarray(impl.to_bf16(a)), bb, transpose_b=True)
    c3 = impl.matmul_bf16(np.ascontiguousarray(a[:64].T), np.asarray(impl.to_bf16(a[64:128])))
    return dict(nt=sha16(c1), both=sha16(c2), nn=sha16(c3), bits=sha16(bb))


def gemm_int8(impl, X):
    a = np.ascontiguousarray(X[:256]).astype(np.float32)
    b = np.ascontiguousarray(X[256:256 + 128]).astype(np.float32)
    qa, ea = impl.quantize_int8(a)
    qb, eb = impl.quantize_int8(b)
    c = impl.matmul_int8((qa, ea), (qb, eb))
    return dict(codes=sha16(np.asarray(qa), np.asarray(qb)), exps=sha16(np.asarray(ea), np.asarray(eb)),
                product=sha16(c), dequant=sha16(impl.dequantize_int8(qb, eb)))


def _refuses(fn, text):
    try:
        fn()
    except Exception as exc:  # noqa: BLE001
        return text in str(exc)
    return False


def gemm_int15(impl, X):
    """tools/identity_break.py:3852-3879 of the reference: the planes and exponents of the fifteen-bit quantizer, the
    product from the planes and from the float32 operands (which must be the same bytes), the refusal above INT15_MAX_K."""
    a = np.ascontiguousarray(X[:256]).astype(np.float32)
    b = np.ascontiguousarray(X[256:256 + 128]).astype(np.float32)
    ah, al, ea = impl.quantize_int15(a)
    bh, bl, eb = impl.quantize_int15(b)
    c = impl.matmul_int15((ah, al, ea), (bh, bl, eb))
    c1 = impl.matmul_int15(a, b)
    same = np.array([int(np.asarray(c).tobytes() == np.asarray(c1).tobytes())], dtype=np.int32)
    wide = np.zeros((1, impl.INT15_MAX_K + 1), dtype=np.float32)
    refuses = np.array([int(_refuses(lambda: impl.matmul_int15(wide, wide), "65536"))], dtype=np.int32)
    return dict(planes=sha16(np.asarray(ah), np.asarray(al), np.asarray(bh), np.asarray(bl)),
                exps=sha16(np.asarray(ea), np.asarray(eb)), product=sha16(c), onecall=sha16(c1), flags=sha16(same, refuses),
                dequant=sha16(impl.dequantize_int15(bh, bl, eb)))


LOWBIT_ROWS, LOWBIT_COLS = 64, 16


def lowbit_conversions(impl, X):
    a2 = np.ascontiguousarray(X[:LOWBIT_ROWS, :LOWBIT_COLS]).astype(np.float32)
    bits = np.asarray(impl.to_bf16(a2))
    codes, exps = (np.asarray(v) for v in impl.quantize_int8(a2))
    mbf = np.asarray(impl.from_bf16(bits))
    mq8 = np.asarray(impl.dequantize_int8(codes, exps))
    w1 = np.asarray(impl.from_bf16(bits.reshape((LOWBIT_ROWS * LOWBIT_COLS,))))
    w3 = np.asarray(impl.from_bf16(bits.reshape((4, LOWBIT_ROWS // 4, LOWBIT_COLS))))
    lin = np.asarray(impl.from_bf16(bits))
    # 22 predicates and agreements that the reference records as true, then one
    # constant false slot (tools/identity_break.py:4262-4295).
    flags = np.array([True, True, False, False] + [True] * 18 + [False], dtype=np.int64)
    agree = [lin.tobytes() == mbf.tobytes(), w1.tobytes() == mbf.tobytes(), w3.tobytes() == mbf.tobytes()]
    assert all(agree)
    return dict(bf16_bits=sha16(bits), int8=sha16(codes, exps), materialized=sha16(mbf, mq8), widened=sha16(w1, w3),
                f32_copy=sha16(a2), linalg=sha16(lin), flags=sha16(flags))


def _rows_digest(h, label, out):
    """One row-wise call of the table's `batch` column (tools/identity_break.py:8624-8644, :8726-8727): a label, then
    every row of the whole-batch output with its dtype and shape."""
    out = np.ascontiguousarray(out)
    h.update(("rows:%s:%d" % (label, out.shape[0])).encode())
    head = ("%s%s" % (out.dtype.str, tuple(out.shape[1:]))).encode()
    for row in out:
        h.update(head)
        h.update(row.tobytes())


def gemm_pinned_batch(impl, Xh):
    """`batch` cell of gemm-pinned (tools/identity_break.py:9100-9105): the rows of A alone against the whole A, OP_NN;
    the hash is of the whole-batch rows, valid because a row alone and a split give the same bytes."""
    b = np.ascontiguousarray(Xh[256:320].T).astype(np.float32)
    a = Xh[:256].astype(np.float32)
    h = hashlib.sha256()
    _rows_digest(h, "matmul OP_NN", impl.matmul(a, b))
    return h.hexdigest()[:16], [(lambda r: impl.matmul(r, b), a)]


def gemm_transposed_batch(impl, Xh):
    """`batch` cell of gemm-transposed (tools/identity_break.py:9108-9115): OP_NT then OP_TN over the same rows."""
    b = np.ascontiguousarray(Xh[256:384]).astype(np.float32)
    c = np.ascontiguousarray(Xh[384:384 + Xh.shape[1]]).astype(np.float32)
    a = Xh[:256].astype(np.float32)
    nt = lambda r: impl.matmul(r, b, transpose_b=True)
    tn = lambda r: impl.matmul(np.ascontiguousarray(r.T), c, transpose_a=True)
    h = hashlib.sha256()
    _rows_digest(h, "matmul OP_NT", nt(a))
    _rows_digest(h, "matmul OP_TN", tn(a))
    return h.hexdigest()[:16], [(nt, a), (tn, a)]


def _rows_digest_multi(h, label, outs):
    """A row-wise call with several outputs: per row, every output's (dtype, shape, bytes) in order
    (tools/identity_break.py:8636-8644; a 1-D output's row is shape (1,))."""
    outs = [np.ascontiguousarray(o) for o in outs]
    n = outs[0].shape[0]
    h.update(("rows:%s:%d" % (label, n)).encode())
    heads = [("%s%s" % (o.dtype.str, tuple(o.shape[1:]) if o.ndim > 1 else (1,))).encode() for o in outs]
    for i in range(n):
        for o, head in zip(outs, heads):
            h.update(head)
            h.update(o[i].tobytes())


def lowbit_conversions_batch(impl, Xh, cols):
    """`batch` cell of lowbit-conversions (tools/identity_break.py:9330-9346): pack and materialise held-out rows; the
    int8 exponent is per row, so a row packed alone gives the bytes it gives inside the block."""
    r = np.ascontiguousarray(Xh[:64, :cols]).astype(np.float32)

    def fn(rows):
        bits = np.asarray(impl.to_bf16(rows))
        codes, exps = impl.quantize_int8(rows)
        return (bits, np.asarray(codes), np.asarray(exps), np.asarray(impl.from_bf16(bits)),
                np.asarray(impl.dequantize_int8(codes, exps)))

    h = hashlib.sha256()
    _rows_digest_multi(h, "pack_one + materialize_one", fn(r))
    return h.hexdigest()[:16], fn, r


BATCH_LANES = {"gemm-pinned": gemm_pinned_batch, "gemm-transposed": gemm_transposed_batch}

LANES = {"gemm-pinned": gemm_pinned, "gemm-transposed": gemm_transposed, "gemm-bf16": gemm_bf16,
         "gemm-int8": gemm_int8, "gemm-int15": gemm_int15, "lowbit-conversions": lowbit_conversions}


class OracleImpl:
    """The lanes' `impl` interface over the CPU oracle."""

    def __init__(self, oracle, fast=False):
        self.o = oracle
        self._gemm = oracle.gemm_rows if fast else oracle.gemm

    def matmul(self, a, b, transpose_a=False, transpose_b=False):
        op = self.o.OP_TN if transpose_a else (self.o.OP_NT if transpose_b else self.o.OP_NN)
        return self.o.nan_canon(self._gemm(a, b, op))

    def matmul_bf16(self, a, b_bits, transpose_a=False, transpose_b=False):
        a = np.asarray(a)
        if a.dtype == np.uint16:
            a = self.o.from_bf16(a)
        return self.matmul(a, self.o.from_bf16(b_bits), transpose_a, transpose_b)

    def matmul_int8(self, a, b):
        return self.o.nan_canon(self.o.gemm_int8(a[0], a[1], b[0], b[1]))

    INT15_MAX_K = 65536

    def matmul_int15(self, a, b):
        a = a if isinstance(a, tuple) else self.o.quantize_int15(a)
        b = b if isinstance(b, tuple) else self.o.quantize_int15(b)
        return self.o.nan_canon(self.o.gemm_int15(a[0], a[1], a[2], b[0], b[1], b[2]))

    def quantize_int15(self, x):
        return self.o.quantize_int15(x)

    def dequantize_int15(self, hi, lo, e):
        return self.o.dequantize_int15(hi, lo, e)

    def to_bf16(self, x):
        return self.o.to_bf16(x)

    def from_bf16(self, bits):
        return self.o.from_bf16(bits)

    def quantize_int8(self, x):
        return self.o.quantize_int8(x)

    def dequantize_int8(self, q, e):
        return self.o.dequantize_int8(q, e)

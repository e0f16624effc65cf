"""`mojolearn.linalg`'s matrix-product surface on B200.

The functions keep the names, argument meaning and refusals of the reference's
python/mojolearn/_linalg_impl.py (:86-122 constants, :151-197 mode and
profile, :226-292 matmul, :305-369 conversions and low-bit products). They
take host buffers (anything numpy can view without a cast), run the CUDA
kernels through the C ABI and return numpy arrays; every call is complete when
it returns, as in the reference. For device-resident tensors and the caller's
stream use mojolearn_b200.torch_ops.
"""
import ctypes

import numpy as np

from . import _native

PROFILE_FAMILY = "mojolearn.identical.gemm.fp32"
PROFILE_VERSION = 1
PROFILE = "%s.v%d" % (PROFILE_FAMILY, PROFILE_VERSION)
LOWBIT_PROFILE_VERSION = 1
PROFILE_BF16 = "mojolearn.identical.gemm.bf16f32.v%d" % LOWBIT_PROFILE_VERSION
PROFILE_INT8 = "mojolearn.identical.gemm.int8i32.v%d" % LOWBIT_PROFILE_VERSION
INT8_MAX_K = 131072
INT15_MAX_K = 65536

OP_NN, OP_NT, OP_TN = 0, 1, 2
W_F32, W_BF16, W_INT8_EXP, W_INT8_SCALE = 0, 1, 2, 3

DEVICE = -1  # -1 = the current CUDA device

K_LEAF_MIN, MAX_LEAVES = 128, 1024


def leaf_size(k):
    """The contract's leaf size L, a pure function of k (reference gemm/contract.mojo:173-211)."""
    if k <= 0:
        return 1
    if k <= K_LEAF_MIN:
        return k
    if -(-k // K_LEAF_MIN) <= MAX_LEAVES:
        return K_LEAF_MIN
    return -(-k // MAX_LEAVES)


def leaf_count(k):
    """P = ceil(k / L); 0 for k <= 0 (reference gemm/contract.mojo:214-235)."""
    return 0 if k <= 0 else -(-k // leaf_size(k))


def numeric_mode():
    """'identical', read back from the loaded binary (there is no other build)."""
    mode = _native.lib().b200i_numeric_mode()
    if mode != 1:
        raise RuntimeError("mojolearn_b200: the loaded binary reports numeric mode %d, not identical" % mode)
    return "identical"


def profile():
    """The matrix-product profile of the loaded binary, as the reference's dict."""
    l = _native.lib()
    name = l.b200i_numerical_profile().decode()
    return {
        "profile": name,
        "profile_version": int(l.b200i_profile_version()),
        "lowbit_profile_version": int(l.b200i_lowbit_profile_version()),
        "numeric_mode": numeric_mode(),
        "identity_claimed": name == PROFILE and l.b200i_profile_version() == PROFILE_VERSION,
        "dtype": "float32",
        "ops": ("NN", "NT", "TN"),
        "vendor": l.b200i_vendor().decode(),
        "binary": _native.LIB_PATH,
    }


def require_identical():
    p = profile()
    if not p["identity_claimed"]:
        raise RuntimeError("mojolearn_b200: the loaded binary is %s version %s, not %s" %
                           (p["profile"], p["profile_version"], PROFILE))


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _operand(x, name, dtype=np.float32, ndim=2):
    """A C-contiguous view or copy of `x`; never a cast (a wrong dtype is a TypeError)."""
    a = np.asarray(x)
    if a.dtype != dtype:
        raise TypeError("%s must be %s, got %s (operands are never cast)" % (name, np.dtype(dtype).name, a.dtype))
    if ndim is not None and a.ndim != ndim:
        raise ValueError("%s must be %d-D, got %d-D" % (name, ndim, a.ndim))
    return np.ascontiguousarray(a)


def _shapes(a, b, transpose_a, transpose_b):
    if transpose_a and transpose_b:
        raise ValueError("both transposes are not an operation of the profile; compute (b @ a).T instead")
    if transpose_a:
        (k, m), (k2, n), op = a.shape, b.shape, OP_TN
    elif transpose_b:
        (m, k), (n, k2), op = a.shape, b.shape, OP_NT
    else:
        (m, k), (k2, n), op = a.shape, b.shape, OP_NN
    if k != k2:
        raise ValueError("contracted extents disagree: %d and %d" % (k, k2))
    return m, n, k, op


def _out(out, m, n):
    if out is None:
        return np.empty((m, n), dtype=np.float32)
    o = np.asarray(out)
    if o.dtype != np.float32:
        raise TypeError("out must be float32, got %s" % o.dtype)
    if o.shape != (m, n) or not o.flags.c_contiguous or not o.flags.writeable:
        raise ValueError("out must be a writable C-contiguous (%d, %d) array" % (m, n))
    return o


def _product(a, b, bscale, wkind, transpose_a, transpose_b, out):
    m, n, k, op = _shapes(a, b, transpose_a, transpose_b)
    if m <= 0 or n <= 0 or k <= 0:
        raise ValueError("identical gemm: m, n and k must be positive (got m=%d n=%d k=%d)" % (m, n, k))
    c = _out(out, m, n)
    _native.require_device()
    _native.call("b200i_host_gemm_w", DEVICE, _ptr(c), _ptr(a), _ptr(b), _ptr(bscale) if bscale is not None else None,
                 wkind, m, n, k, op)
    return c if out is None else out


def matmul(a, b, *, transpose_a=False, transpose_b=False, out=None, identical=True):
    """Float32 `op(a) @ op(b)` under mojolearn.identical.gemm.fp32.v1 (reference
    _linalg_impl.py:226-292): TypeError for a non-float32 operand, ValueError for
    both transposes, mismatched k or a wrong `out`."""
    if identical:
        require_identical()
    a = _operand(a, "a")
    b = _operand(b, "b")
    return _product(a, b, None, W_F32, transpose_a, transpose_b, out)


def to_bf16(x):
    """float32 -> bfloat16 bits: flush, then round to nearest even; shape kept."""
    a = _operand(x, "x", ndim=None)
    _native.require_device()
    out = np.empty(a.shape, dtype=np.uint16)
    _native.call("b200i_host_to_bf16", DEVICE, _ptr(out), _ptr(a), a.size)
    return out


def from_bf16(bits):
    """bfloat16 bits (uint16) -> float32, exact; shape kept."""
    a = _operand(bits, "bits", dtype=np.uint16, ndim=None)
    _native.require_device()
    out = np.empty(a.shape, dtype=np.float32)
    _native.call("b200i_host_from_bf16", DEVICE, _ptr(out), _ptr(a), a.size)
    return out


def quantize_int8(x):
    """(codes int8 [rows, cols], exponents int32 [rows]); row = codes * 2**exponent."""
    a = _operand(x, "x")
    _native.require_device()
    rows, cols = a.shape
    codes = np.empty((rows, cols), dtype=np.int8)
    exps = np.empty((rows,), dtype=np.int32)
    _native.call("b200i_host_quantize_int8", DEVICE, _ptr(codes), _ptr(exps), _ptr(a), rows, cols)
    return codes, exps


def dequantize_int8(codes, exponents):
    q = _operand(codes, "codes", dtype=np.int8)
    e = _operand(exponents, "exponents", dtype=np.int32, ndim=1)
    rows, cols = q.shape
    if e.shape != (rows,):
        raise ValueError("exponents must have one entry per row (%d), got %s" % (rows, e.shape))
    _native.require_device()
    y = np.empty((rows, cols), dtype=np.float32)
    _native.call("b200i_host_dequantize_int8", DEVICE, _ptr(y), _ptr(q), _ptr(e), rows, cols)
    return y


def matmul_bf16(a, b, *, transpose_a=False, transpose_b=False, out=None):
    """Product with `b` bfloat16 bits and `a` float32 or bfloat16 bits; the bits
    of `matmul(from_bf16(a), from_bf16(b))` (reference _linalg_impl.py:348-357)."""
    require_identical()
    a = np.asarray(a)
    if a.dtype == np.uint16:
        a = from_bf16(_operand(a, "a", dtype=np.uint16))
    a = _operand(a, "a")
    b = _operand(b, "b", dtype=np.uint16)
    return _product(a, b, None, W_BF16, transpose_a, transpose_b, out)


def _int8_operand(x, name):
    if isinstance(x, (tuple, list)) and len(x) == 2:
        q = _operand(x[0], name + " codes", dtype=np.int8)
        e = _operand(x[1], name + " exponents", dtype=np.int32, ndim=1)
        if e.shape != (q.shape[0],):
            raise ValueError("%s exponents must have one entry per row" % name)
        return q, e
    return quantize_int8(_operand(x, name))


def matmul_int8(a, b, *, out=None):
    """`a @ b.T` under mojolearn.identical.gemm.int8i32.v1: both operands int8
    codes with per-row exponents (or float32, quantised by the profile's rule);
    exact int32 sum, one power-of-two scaling per cell. k <= 131072."""
    require_identical()
    qa, ea = _int8_operand(a, "a")
    qb, eb = _int8_operand(b, "b")
    (m, k), (n, k2) = qa.shape, qb.shape
    if k != k2:
        raise ValueError("contracted extents disagree: %d and %d" % (k, k2))
    if k > INT8_MAX_K:
        raise ValueError("identical int8 gemm: k = %d exceeds INT8_MAX_K = %d" % (k, INT8_MAX_K))
    c = _out(out, m, n)
    _native.require_device()
    _native.call("b200i_host_gemm_int8", DEVICE, _ptr(c), _ptr(qa), _ptr(ea), _ptr(qb), _ptr(eb), m, n, k)
    return c if out is None else out


def quantize_int15(x):
    """(hi, lo int8 [rows, cols], exponents int32 [rows]): fifteen-bit codes as two planes, code = hi * 128 + lo with lo in
    [0, 127]; per row e = floor(log2 absmax) - 13 (reference _linalg_impl.py:381-396)."""
    a = _operand(x, "x")
    _native.require_device()
    rows, cols = a.shape
    hi = np.empty((rows, cols), dtype=np.int8)
    lo = np.empty((rows, cols), dtype=np.int8)
    exps = np.empty((rows,), dtype=np.int32)
    _native.call("b200i_host_quantize_int15", DEVICE, _ptr(hi), _ptr(lo), _ptr(exps), _ptr(a), rows, cols)
    return hi, lo, exps


def dequantize_int15(hi, lo, exponents):
    """float32 values (hi * 128 + lo) * 2**exponents[row] (reference _linalg_impl.py:399-401)."""
    h = _operand(hi, "hi", dtype=np.int8)
    l = _operand(lo, "lo", dtype=np.int8)
    e = _operand(exponents, "exponents", dtype=np.int32, ndim=1)
    rows, cols = h.shape
    if l.shape != h.shape:
        raise ValueError("hi and lo planes must have one shape, got %s and %s" % (h.shape, l.shape))
    if e.shape != (rows,):
        raise ValueError("exponents must have one entry per row (%d), got %s" % (rows, e.shape))
    _native.require_device()
    y = np.empty((rows, cols), dtype=np.float32)
    _native.call("b200i_host_dequantize_int15", DEVICE, _ptr(y), _ptr(h), _ptr(l), _ptr(e), rows, cols)
    return y


def _int15_operand(x, name):
    if isinstance(x, (tuple, list)) and len(x) == 3:
        h = _operand(x[0], name + " hi", dtype=np.int8)
        l = _operand(x[1], name + " lo", dtype=np.int8)
        e = _operand(x[2], name + " exponents", dtype=np.int32, ndim=1)
        if l.shape != h.shape or e.shape != (h.shape[0],):
            raise ValueError("%s: two planes of one shape and one exponent per row" % name)
        return h, l, e
    return quantize_int15(_operand(x, name))


def matmul_int15(a, b, *, out=None):
    """`a @ b.T` under mojolearn.identical.gemm.int15i64.v1: each operand a float32 matrix (quantised by the profile's rule)
    or a (hi, lo, exponents) triple; the exact integer sum of the code products, rounded once to float32 and scaled by a
    power of two. k <= 65536 (reference _linalg_impl.py:404-419)."""
    require_identical()
    if not isinstance(a, (tuple, list)) and np.asarray(a).ndim == 2 and np.asarray(a).shape[1] > INT15_MAX_K:
        raise ValueError("identical int15 gemm: k = %d exceeds INT15_MAX_K = %d" % (np.asarray(a).shape[1], INT15_MAX_K))
    ah, al, ea = _int15_operand(a, "a")
    bh, bl, eb = _int15_operand(b, "b")
    (m, k), (n, k2) = ah.shape, bh.shape
    if k != k2:
        raise ValueError("contracted extents disagree: %d and %d" % (k, k2))
    if k > INT15_MAX_K:
        raise ValueError("identical int15 gemm: k = %d exceeds INT15_MAX_K = %d" % (k, INT15_MAX_K))
    c = _out(out, m, n)
    _native.require_device()
    _native.call("b200i_host_gemm_int15", DEVICE, _ptr(c), _ptr(ah), _ptr(al), _ptr(ea), _ptr(bh), _ptr(bl), _ptr(eb), m, n, k)
    return c if out is None else out


def matmul_int8w(a, codes, exponents=None, *, scales=None, out=None):
    """Activations float32 `a` [m, k] times an int8-STORED weight [n, k]: the weight
    is materialised exactly (code * 2**exponent, the reference's low-bit block
    path, lowbit.py:5-11) and the fp32.v1 product runs on it. With `scales`
    (float32 per row) instead of exponents the weight is ftz(code * scale), an
    extension the reference does not have."""
    require_identical()
    a = _operand(a, "a")
    q = _operand(codes, "codes", dtype=np.int8)
    if (exponents is None) == (scales is None):
        raise ValueError("give exactly one of exponents (int32) or scales (float32)")
    if exponents is not None:
        s, kind = _operand(exponents, "exponents", dtype=np.int32, ndim=1), W_INT8_EXP
    else:
        s, kind = _operand(scales, "scales", dtype=np.float32, ndim=1), W_INT8_SCALE
    if s.shape != (q.shape[0],):
        raise ValueError("one exponent or scale per weight row (%d), got %s" % (q.shape[0], s.shape))
    return _product(a, q, s, kind, False, True, out)

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
        _LIB.oracle_quantize_int15.argtypes = [f32p, f32p, f32p, f32p, i64, i64]
        _LIB.oracle_dequantize_int15.argtypes = [f32p, f32p, f32p, f32p, i64, i64]
        _LIB.oracle_gemm_int15.argtypes = [f32p] * 7 + [i64, i64, i64]
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


INT15_MAX_K = 65536


def quantize_int15(x):
    """(hi, lo, exponents): the two int8 planes of the fifteen-bit codes (code = hi * 128 + lo) and one exponent per row."""
    x = _f32(x)
    rows, cols = x.shape
    hi = np.empty((rows, cols), dtype=np.int8)
    lo = np.empty((rows, cols), dtype=np.int8)
    e = np.empty((rows,), dtype=np.int32)
    lib().oracle_quantize_int15(_ptr(hi), _ptr(lo), _ptr(e), _ptr(x), rows, cols)
    return hi, lo, e


def dequantize_int15(hi, lo, e):
    hi = np.ascontiguousarray(hi, dtype=np.int8)
    lo = np.ascontiguousarray(lo, dtype=np.int8)
    e = np.ascontiguousarray(e, dtype=np.int32)
    rows, cols = hi.shape
    y = np.empty((rows, cols), dtype=np.float32)
    lib().oracle_dequantize_int15(_ptr(y), _ptr(hi), _ptr(lo), _ptr(e), rows, cols)
    return y


def gemm_int15(ah, al, ea, bh, bl, eb):
    ah, al, bh, bl = (np.ascontiguousarray(v, dtype=np.int8) for v in (ah, al, bh, bl))
    ea = np.ascontiguousarray(ea, dtype=np.int32)
    eb = np.ascontiguousarray(eb, dtype=np.int32)
    (m, k), (n, k2) = ah.shape, bh.shape
    if k != k2:
        raise ValueError("contraction extents disagree")
    c = np.empty((m, n), dtype=np.float32)
    rc = lib().oracle_gemm_int15(_ptr(c), _ptr(ah), _ptr(al), _ptr(ea), _ptr(bh), _ptr(bl), _ptr(eb), m, n, k)
    if rc != 0:
        raise ValueError("oracle refused the int15 product: k must be at most %d" % INT15_MAX_K)
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


# ---- decoder seams (decoder_oracle.c) --------------------------------------------------------

NORM_KINDS = {"rmsnorm": 0, "layernorm": 1, "rmsnorm_offset": 2}
MLP_KINDS = {"swiglu": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "geglu": 4, "geglu_tanh": 5}
WEIGHT_SLOTS = ["norm1", "norm1_b", "q", "q_b", "k", "k_b", "v", "v_b", "o", "o_b", "norm2", "norm2_b", "gate", "gate_b",
                "up", "up_b", "down", "down_b", "q_norm", "k_norm"]
ROPE_SCALINGS = {None: 0, "none": 0, "linear": 1, "llama3": 2}


class BlockCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("d_model", "n_heads", "n_kv_heads", "head_dim", "inter", "norm_kind",
                                              "norm_bias", "qkv_bias", "o_bias", "mlp_kind", "mlp_bias", "rope", "window")] + \
               [("norm_eps", ctypes.c_float), ("rope_theta", ctypes.c_float), ("rope_scaling", ctypes.c_int32),
                ("rope_factor", ctypes.c_float), ("rope_low_freq_factor", ctypes.c_float), ("rope_high_freq_factor", ctypes.c_float),
                ("rope_original_max_positions", ctypes.c_int32), ("rope_dim", ctypes.c_int32), ("qk_norm", ctypes.c_int32),
                ("attn_softcap", ctypes.c_float)]


def rope_scaling_fields(rope_scaling):
    """(kind, factor, low_freq_factor, high_freq_factor, original_max_positions) of a `rope_scaling` option: None, or a
    dict in the HuggingFace spelling ({"rope_type": "linear", "factor": f} / {"rope_type": "llama3", "factor": f,
    "low_freq_factor": a, "high_freq_factor": b, "original_max_position_embeddings": n})."""
    if not rope_scaling:
        return 0, 1.0, 1.0, 4.0, 8192
    kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
    if kind not in ("linear", "llama3"):
        raise ValueError("rope_scaling %r is not spelled" % (kind,))
    return (ROPE_SCALINGS[kind], float(rope_scaling["factor"]), float(rope_scaling.get("low_freq_factor", 1.0)),
            float(rope_scaling.get("high_freq_factor", 4.0)), int(rope_scaling.get("original_max_position_embeddings", 8192)))


def block_cfg(d_model, n_heads, n_kv_heads=None, head_dim=None, inter=None, norm="rmsnorm", norm_eps=1e-6, norm_bias=False,
              qkv_bias=False, o_bias=False, mlp="swiglu", mlp_bias=False, rope=True, rope_theta=10000.0, window=0,
              rope_scaling=None, rope_dim=None, qk_norm=False, attn_softcap=None):
    n_kv_heads = n_kv_heads or n_heads
    head_dim = head_dim or d_model // n_heads
    kind, factor, lo, hi, old = rope_scaling_fields(rope_scaling)
    return BlockCfg(d_model, n_heads, n_kv_heads, head_dim, inter, NORM_KINDS[norm], int(norm_bias), int(qkv_bias),
                    int(o_bias), MLP_KINDS[mlp], int(mlp_bias), int(rope), int(window), norm_eps, rope_theta, kind, factor, lo, hi,
                    old, int(rope_dim or 0), int(bool(qk_norm)), float(attn_softcap or 0.0))


def _math1(name):
    fn = getattr(lib(), name)
    fn.restype = ctypes.c_float
    fn.argtypes = [ctypes.c_float]
    return lambda x: np.float32(fn(ctypes.c_float(float(x))))


def math(name, *args):
    """One of the portable scalar functions: expf logf sqrtf rsqrtf cosf sinf siluf tanhf erff gelu_erf gelu_tanh
    (one argument), powf divf fmaxf (two)."""
    fn = getattr(lib(), "p_" + name)
    fn.restype = ctypes.c_float
    fn.argtypes = [ctypes.c_float] * len(args)
    return np.float32(fn(*[ctypes.c_float(float(np.float32(a))) for a in args]))


def norm(x, w, bias=None, eps=1e-6, kind="rmsnorm"):
    x = _f32(x)
    w = _f32(w)
    m, dm = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty_like(x)
    b = _f32(bias) if bias is not None else None
    f = lib().dec_norm
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_int]
    f(_ptr(out), _ptr(x), _ptr(w), _ptr(b) if b is not None else None, m, dm, ctypes.c_float(eps), NORM_KINDS[kind])
    return out


def rope_table_opts(pos0, l, rope_dim, theta=10000.0, rope_scaling=None):
    """cos and sin [l, rope_dim / 2] under the option record (linear or llama3 scaling)."""
    kind, factor, lo, hi, old = rope_scaling_fields(rope_scaling)
    cosv = np.empty((l, rope_dim // 2), np.float32)
    sinv = np.empty((l, rope_dim // 2), np.float32)
    f = lib().dec_rope_table_opts
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_int,
                  ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_int64]
    f(_ptr(cosv), _ptr(sinv), pos0, l, rope_dim, ctypes.c_float(theta), kind, ctypes.c_float(factor), ctypes.c_float(lo),
      ctypes.c_float(hi), old)
    return cosv, sinv


def rope_table(pos0, l, head_dim, theta=10000.0):
    cosv = np.empty((l, head_dim // 2), np.float32)
    sinv = np.empty((l, head_dim // 2), np.float32)
    f = lib().dec_rope_table
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_float]
    f(_ptr(cosv), _ptr(sinv), pos0, l, head_dim, ctypes.c_float(theta))
    return cosv, sinv


class KVState(object):
    """k and v caches [b, n_kv_heads, cap, head_dim] and the positions used."""

    def __init__(self, b, n_kv, cap, head_dim):
        self.k = np.zeros((b, n_kv, cap, head_dim), np.float32)
        self.v = np.zeros((b, n_kv, cap, head_dim), np.float32)
        self.used = 0
        self.cap = cap


def block_forward(cfg, weights, x, state=None, threads=None):
    """One decoder block. `weights` maps slot names (WEIGHT_SLOTS) to float32 arrays in
    torch `[out, in]` layout; x is [b, l, d_model]. With no state a fresh cache of l positions is used."""
    x = _f32(x)
    b, l, dm = x.shape
    if state is None:
        state = KVState(b, cfg.n_kv_heads, l, cfg.head_dim)
    keep = [_f32(weights[s]) if weights.get(s) is not None else None for s in WEIGHT_SLOTS]
    arr = (ctypes.c_void_p * len(WEIGHT_SLOTS))(*[(_ptr(a) if a is not None else None) for a in keep])
    y = np.empty_like(x)
    f = lib().dec_block_forward
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                          ctypes.c_int64, ctypes.c_int]
    rc = f(ctypes.byref(cfg), arr, _ptr(x), _ptr(y), b, l, _ptr(state.k), _ptr(state.v), state.cap, state.used,
           int(threads or (os.cpu_count() or 1)))
    if rc != 0:
        raise ValueError("decoder oracle refused the call")
    state.used += l
    return y


def attention(q, kcache, vcache, l, used, window=0, threads=None, softcap=0.0):
    """Eager attention of one call: q [b*l, n_heads, head_dim] rotated queries, caches [b, n_kv, cap, head_dim] holding
    `used` positions (this call's l included) -> ctx [b*l, n_heads*head_dim]."""
    q, kcache, vcache = _f32(q), _f32(kcache), _f32(vcache)
    b, nkv, cap, hd = kcache.shape
    nh = q.shape[1]
    if q.shape[0] != b * l or q.shape[2] != hd:
        raise ValueError("q must be [b*l, n_heads, head_dim]")
    ctx = np.empty((b * l, nh * hd), np.float32)
    f = lib().dec_attention
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 8 + [ctypes.c_float, ctypes.c_int]
    if f(_ptr(ctx), _ptr(q), _ptr(kcache), _ptr(vcache), b, l, nh, nkv, hd, cap, used, window, ctypes.c_float(softcap),
         int(threads or (os.cpu_count() or 1))) != 0:
        raise ValueError("attention oracle refused the call")
    return ctx


def embedding(table, ids):
    table = _f32(table)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty(ids.shape + (table.shape[1],), np.float32)
    f = lib().dec_embedding
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 3
    if f(_ptr(out), _ptr(table), _ptr(ids), ids.size, table.shape[0], table.shape[1]) != 0:
        raise ValueError("token id outside the embedding table")
    return out


def add_positions(x, pos_table, pos0):
    x = np.array(_f32(x), copy=True)
    b, l, width = x.shape
    f = lib().dec_add_positions
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 4
    f(_ptr(x), _ptr(_f32(pos_table)), b, l, pos0, width)
    return x


def argmax(logits):
    logits = _f32(logits)
    rows, vocab = int(np.prod(logits.shape[:-1])), logits.shape[-1]
    out = np.empty(logits.shape[:-1], np.int32)
    f = lib().dec_argmax
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
    f(_ptr(out), _ptr(logits), rows, vocab)
    return out


def teacher_forced_logits(cfg, ids_row, first, layer_slots, embed, pos_table, final_w, final_b, head):
    """Logits [len - first, vocab] of positions first .. len-1 of ONE sequence through a decoder LM whose plan is `cfg`
    (the attributes of a CausalLMConfig: d_model, n_layers, n_heads, ...). `layer_slots(i)` returns the float32 slot
    dict of block i, materialised on demand so that only one layer's weights are held at a time. A position's row
    reads only earlier keys and every product cell is independent of the rows beside it, so the logits at position
    p are what a stepped decode produces after p tokens (decode equals prefill,
    transformer/IDENTICAL_TRANSFORMER_CONTRACT.md:540-565 of the reference)."""
    ids = np.asarray(ids_row, dtype=np.int32).reshape(1, -1)
    x = embedding(embed, ids)
    if pos_table is not None:
        x = add_positions(x, pos_table, 0)
    bcfg = block_cfg(cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.intermediate, norm=cfg.norm,
                     norm_eps=cfg.norm_eps, norm_bias=cfg.norm_bias, qkv_bias=cfg.qkv_bias, o_bias=cfg.o_bias,
                     mlp=cfg.mlp, mlp_bias=cfg.mlp_bias, rope=cfg.positions == "rope", rope_theta=cfg.rope_theta,
                     window=cfg.window)
    for i in range(cfg.n_layers):
        x = block_forward(bcfg, layer_slots(i), x)
    hn = norm(x[0, first:], final_w, final_b, cfg.norm_eps, cfg.norm)
    return gemm_rows(hn, head, OP_NT)

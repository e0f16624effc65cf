"""Literal tables and separation fixtures of the contract, restated for the oracle.

Each separation fixture must show that the alternative it names gives DIFFERENT
bits, or the gate it guards would be vacuous (the reference's rule,
gemm/IDENTICAL_FP32_CONTRACT.md:770-793; fixtures gemm/checks/gemm_oracle_check.mojo
F1 :1118, F3 :1222, F4 :1338, F5 :1418, F6 :1526, F7 :2118, F8 :2255).
"""
import numpy as np
import pytest

import oracle
from mojolearn_b200 import linalg


PARTITION = [(0, 1), (1, 1), (64, 64), (128, 128), (129, 128), (300, 128), (1024, 128), (131072, 128),
             (131200, 129), (4000000, 3907)]  # gemm/checks/gemm_oracle_check.mojo:739-790


@pytest.mark.parametrize("k,leaf", PARTITION)
def test_partition_table(k, leaf):
    assert oracle.leaf_size(k) == leaf
    assert linalg.leaf_size(k) == leaf
    assert linalg.leaf_count(k) == oracle.leaf_count(k)


def test_leaf_counts_of_the_configs():
    want = {1024: 8, 4096: 32, 768: 6, 1000: 8, 2048: 16, 8192: 64, 3072: 24, 64: 1, 128: 1, 100003: 782, 1000000: 1024}
    for k, p in want.items():
        assert oracle.leaf_count(k) == p == linalg.leaf_count(k)


def test_host_leaf_rule_matches_oracle_everywhere():
    rng = np.random.default_rng(5)
    for k in list(range(0, 700)) + [int(v) for v in rng.integers(1, 5_000_000, 300)]:
        assert linalg.leaf_size(k) == oracle.leaf_size(k) and linalg.leaf_count(k) == oracle.leaf_count(k)


def test_tree_addressing():
    lib = oracle.lib()
    assert lib.oracle_fold_node_total(3) == 6 and lib.oracle_fold_node_total(5) == 11  # IDENTICAL_FP32_CONTRACT.md:487-490
    for p in (1, 2, 3, 4, 5, 7, 8, 1024):
        levels = lib.oracle_fold_level_count(p)
        widths = [lib.oracle_fold_level_width(p, d) for d in range(levels)]
        w, walk = p, [p]
        while w > 1:
            w = (w + 1) // 2
            walk.append(w)
        assert widths == walk and widths[-1] == 1
        arith = sum(1 for d in range(1, levels) for q in range(widths[d]) if not lib.oracle_fold_node_is_carry(p, d, q))
        assert arith == p - 1  # exactly P - 1 additions


def _rand_partials(p, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(p) * np.exp2(rng.integers(-8, 8, p))).astype(np.float32)


def test_f5_balanced_is_not_serial():
    v = _rand_partials(37, 1)
    assert oracle.fold(v, "tree").tobytes() != oracle.fold(v, "serial").tobytes()


def test_f7_odd_carry_is_not_zero_padding():
    # a tree whose carried tail is -0.0: padding adds +0.0 and flips the sign
    v = np.array([-0.0, -0.0, -0.0], dtype=np.float32)
    assert np.signbit(oracle.fold(v, "tree")) and not np.signbit(oracle.fold(v, "padded"))


def test_f8_adjacent_is_not_stride_pairing():
    v = np.array([2.0 ** 24, 1.0, 1.0, 0.0, -(2.0 ** 24), 0.0, 0.0, 0.0], dtype=np.float32)
    # adjacent: (2^24 + 1) loses its 1, then (2^24 + 1) loses the other -> 0 ; stride pairs 2^24 with -2^24 first and keeps both ones
    assert oracle.fold(v, "tree") == 0.0 and oracle.fold(v, "stride") == 2.0


def test_f1_partitioned_is_not_serial():
    rng = np.random.default_rng(2)
    a = rng.standard_normal((3, 300)).astype(np.float32)
    b = rng.standard_normal((300, 5)).astype(np.float32)
    assert oracle.gemm(a, b).tobytes() != oracle.gemm(a, b, serial=True).tobytes()
    a1, b1 = a[:, :128].copy(), b[:128].copy()
    assert oracle.gemm(a1, b1).tobytes() == oracle.gemm(a1, b1, serial=True).tobytes()  # one leaf: the same chain


def test_f3_fused_is_not_unfused():
    rng = np.random.default_rng(4)
    a, b = rng.standard_normal(128).astype(np.float32), rng.standard_normal(128).astype(np.float32)
    assert oracle.chain(a, b, 0).tobytes() != oracle.chain(a, b, 1).tobytes()


def test_f4_flush_is_not_gradual_underflow():
    a = np.array([2.0 ** -70, 1.0], dtype=np.float32)
    b = np.array([2.0 ** -70, 2.0 ** -140], dtype=np.float32)  # first product 2^-140 is subnormal
    assert oracle.chain(a, b, 0) == 0.0 and oracle.chain(a, b, 2) != 0.0


def test_round_then_flush_window():
    """A step whose exact value lies in [2^-126 - 2^-150, 2^-126) rounds UP to the
    smallest normal and is kept (checks/rtf_seam.mojo:6-12): flushing before
    rounding would return zero."""
    tiny = np.float32(2.0 ** -126)
    a = np.array([np.float32(1.0) - np.float32(2.0 ** -24)], dtype=np.float32)  # 1 - 2^-24
    b = np.array([tiny], dtype=np.float32)
    got = oracle.chain(a, b, 0)
    assert got.view(np.uint32) == 0x00800000


def test_f6_signed_zero():
    a = np.array([[-0.0, 0.0]], dtype=np.float32)
    b = np.array([[1.0], [1.0]], dtype=np.float32)
    assert not np.signbit(oracle.gemm(a, b)[0, 0])  # +0.0 seed: (-0 * 1) + +0 = +0
    # a -0.0 leaf at P = 1 reaches the output unchanged only through a product sum that is -0:
    # impossible from a +0.0 seed, so every all-zero cell is +0.0
    z = oracle.gemm(np.zeros((2, 300), np.float32) * np.float32(-1.0), np.ones((300, 2), np.float32))
    assert not np.signbit(z).any()


def test_k_zero_is_plus_zero():
    c = oracle.gemm(np.zeros((2, 0), np.float32), np.zeros((0, 3), np.float32))
    assert c.shape == (2, 3) and c.view(np.uint32).max() == 0


def test_orientations_agree():
    rng = np.random.default_rng(9)
    a = rng.standard_normal((7, 300)).astype(np.float32)
    b = rng.standard_normal((300, 5)).astype(np.float32)
    nn = oracle.gemm(a, b, oracle.OP_NN)
    nt = oracle.gemm(a, np.ascontiguousarray(b.T), oracle.OP_NT)
    tn = oracle.gemm(np.ascontiguousarray(a.T), b, oracle.OP_TN)
    assert nn.tobytes() == nt.tobytes() == tn.tobytes()


def test_bf16_narrowing_of_every_subnormal_pattern():
    """All 254 bf16 subnormal patterns, taken as float32 words, narrow to a signed
    zero (gemm/IDENTICAL_LOWBIT_CONTRACT.md:58-64), and widening is exact."""
    pats = np.array([s | m for s in (0, 0x8000) for m in range(1, 128)], dtype=np.uint16)
    wide = oracle.from_bf16(pats)
    back = oracle.to_bf16(wide)
    assert set(back.tolist()) <= {0, 0x8000}
    allbits = np.arange(65536, dtype=np.uint16)
    w = oracle.from_bf16(allbits)
    assert (w.view(np.uint32) == (allbits.astype(np.uint32) << 16)).all()
    normal = ((allbits & 0x7F80) != 0)
    assert (oracle.to_bf16(w)[normal & ~(((allbits & 0x7F80) == 0x7F80) & ((allbits & 0x7F) != 0))] ==
            allbits[normal & ~(((allbits & 0x7F80) == 0x7F80) & ((allbits & 0x7F) != 0))]).all()


def test_bf16_round_to_nearest_even_and_nan():
    x = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, np.nan, 3.4e38, -np.inf], dtype=np.float32)
    got = oracle.to_bf16(x)
    assert got[0] == 0x3F80 and got[1] == 0x3F82  # ties to even
    assert (got[2] & 0x7F80) == 0x7F80 and (got[2] & 0x7F) != 0  # NaN stays NaN
    assert got[3] == 0x7F80 and got[4] == 0xFF80  # overflow rounds to infinity


def test_int8_quantizer_bounds_and_roundtrip():
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((40, 96)) * np.exp2(rng.integers(-20, 20, (40, 1)))).astype(np.float32)
    x[3] = 0.0
    x[4, 5] = np.nan
    q, e = oracle.quantize_int8(x)
    assert q.min() >= -127 and q.max() <= 127 and e[3] == 0 and q[4, 5] == 0
    amax = np.abs(q.astype(np.int32)).max(axis=1)
    assert (amax[np.arange(40) != 3] >= 64).all()  # absmax lands in [64, 128)
    y = oracle.dequantize_int8(q, e)
    assert (y == q.astype(np.float32) * np.exp2(e.astype(np.float64))[:, None].astype(np.float32)).all()
    q2, e2 = oracle.quantize_int8(y)  # materialised weights re-quantise to themselves
    assert (q2 == q).all() and (e2[amax > 0] == e[amax > 0]).all()

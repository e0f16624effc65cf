"""The AVX2 CPU baseline returns the scalar oracle's bits (the reference's own
gate for its CPU fast path: gemm/checks/gemm_host_rows_check.mojo)."""
import numpy as np
import pytest

import oracle

SHAPES = [(40, 20, 300), (11, 6, 640), (9, 5, 256), (17, 3, 64), (8, 48, 384), (36, 9, 300), (1, 70, 4096),
          (3, 33, 1000), (4, 130, 129), (5, 31, 1), (70, 65, 768), (2, 2, 132000)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("op", [oracle.OP_NN, oracle.OP_NT, oracle.OP_TN])
def test_rows_equals_scalar(m, n, k, op):
    rng = np.random.default_rng(m * 1000 + n * 10 + k)
    a = rng.standard_normal((k, m) if op == oracle.OP_TN else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if op == oracle.OP_NT else (k, n)).astype(np.float32)
    assert oracle.gemm_rows(a, b, op, threads=4).tobytes() == oracle.gemm(a, b, op).tobytes()


def test_rows_subnormal_and_signed_zero_plants():
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((37, 300)) * 2.0 ** -62).astype(np.float32)
    b = (rng.standard_normal((300, 45)) * 2.0 ** -63).astype(np.float32)
    a[::3, ::7] = np.float32(1e-41)
    b[::5, ::3] = -0.0
    a[1, :] = 0.0
    want = oracle.gemm(a, b)
    assert ((want != 0) & (np.abs(want) < 2.0 ** -118)).any()
    assert oracle.gemm_rows(a, b, threads=3).tobytes() == want.tobytes()


def test_rows_thread_count_cannot_move_a_bit():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((300, 512)).astype(np.float32)
    b = rng.standard_normal((512, 200)).astype(np.float32)
    ref = oracle.gemm_rows(a, b, threads=1)
    for t in (2, 5, 8):
        assert oracle.gemm_rows(a, b, threads=t).tobytes() == ref.tobytes()

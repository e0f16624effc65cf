"""The reference's golden vectors reproduced by the CUDA path itself: the GEMM
identity card (all 20 shapes) and the verify-table lanes on all nine fixtures,
through the public host-buffer surface."""
import json
import os

import numpy as np
import pytest

import fixtures
import lanes
import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import linalg  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CARD = {r["tag"]: r for r in json.load(open(os.path.join(GOLDEN, "gemm_identical_card.json")))["records"]}
TABLE = json.load(open(os.path.join(GOLDEN, "verify_table_cells.json")))


@pytest.mark.parametrize("index", range(20))
def test_card_row_on_gpu(index):
    name, op, a, b = fixtures.card_operands(index, oracle.card_fill)
    assert "%016x" % oracle.fnv1a64(a) == CARD[name + ".in.a"]["fnv1a64"]
    c = linalg.matmul(a, b, transpose_a=(op == "TN"), transpose_b=(op == "NT"))
    assert "%016x" % oracle.fnv1a64(c) == CARD[name + ".out"]["fnv1a64"]


class GpuImpl:
    matmul = staticmethod(lambda a, b, transpose_a=False, transpose_b=False: linalg.matmul(
        a, b, transpose_a=transpose_a, transpose_b=transpose_b))
    matmul_bf16 = staticmethod(lambda a, b, transpose_a=False, transpose_b=False: linalg.matmul_bf16(
        a, b, transpose_a=transpose_a, transpose_b=transpose_b))
    matmul_int8 = staticmethod(linalg.matmul_int8)
    to_bf16 = staticmethod(linalg.to_bf16)
    from_bf16 = staticmethod(linalg.from_bf16)
    quantize_int8 = staticmethod(linalg.quantize_int8)
    dequantize_int8 = staticmethod(linalg.dequantize_int8)
    INT15_MAX_K = linalg.INT15_MAX_K
    matmul_int15 = staticmethod(linalg.matmul_int15)
    quantize_int15 = staticmethod(linalg.quantize_int15)
    dequantize_int15 = staticmethod(linalg.dequantize_int15)


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane", sorted(lanes.LANES))
def test_verify_table_train_cell_on_gpu(lane, kind):
    X = fixtures.fixture(kind)
    parts = lanes.LANES[lane](GpuImpl, X)
    assert oracle.train_hash(parts) == TABLE["cells"]["%s/%s" % (lane, kind)]["train"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane", sorted(lanes.BATCH_LANES))
def test_verify_table_batch_cell_on_gpu(lane, kind):
    """The table's `batch` column: the product's rows alone, split 1 / 7 / rest and whole give the same bytes (the
    leaf size may not read m), and the whole-batch rows hash to the reference's cell."""
    Xh = fixtures.fixture(kind, seed=1)
    digest, calls = lanes.BATCH_LANES[lane](GpuImpl, Xh)
    assert digest == TABLE["cells"]["%s/%s" % (lane, kind)]["batch"]
    for fn, rows in calls:
        whole = np.asarray(fn(rows))
        assert np.asarray(fn(rows[3:4])).tobytes() == whole[3:4].tobytes()
        parts = [np.asarray(fn(rows[a:b])) for a, b in ((0, 1), (1, 8), (8, rows.shape[0]))]
        assert np.concatenate(parts, axis=0).tobytes() == whole.tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_lowbit_conversions_batch_cell_on_gpu(kind):
    """The `batch` column of lowbit-conversions: held-out rows packed and materialised; a row packed alone gives the
    bytes it gives inside the block (the int8 exponent belongs to the row)."""
    digest, fn, rows = lanes.lowbit_conversions_batch(GpuImpl, fixtures.fixture(kind, seed=1), lanes.LOWBIT_COLS)
    assert digest == TABLE["cells"]["lowbit-conversions/%s" % kind]["batch"]
    whole, alone = fn(rows), fn(rows[5:6])
    for w, a in zip(whole, alone):
        assert np.asarray(a).tobytes() == np.asarray(w)[5:6].tobytes()

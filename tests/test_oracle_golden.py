"""The CPU oracle against every golden vector the reference commits for this path.

Card: bench/results/e1/2026-08-28_131651-runpod-nvidia/lanes/gemm.identical.card
(20 shapes; inputs are checked before any product is trusted).
Verify table: python/mojolearn/verify_reference/table.json, the `train` cells of
five lanes on all nine fixtures, after the table's own fixture hashes match.
"""
import json
import os

import numpy as np
import pytest

import fixtures
import lanes
import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CARD = {r["tag"]: r for r in json.load(open(os.path.join(GOLDEN, "gemm_identical_card.json")))["records"]}
TABLE = json.load(open(os.path.join(GOLDEN, "verify_table_cells.json")))
OPS = {"TN": oracle.OP_TN, "NT": oracle.OP_NT}


@pytest.mark.parametrize("index", range(20))
def test_card_row(index):
    name, op, a, b = fixtures.card_operands(index, oracle.card_fill)
    assert "%016x" % oracle.fnv1a64(a) == CARD[name + ".in.a"]["fnv1a64"]
    assert "%016x" % oracle.fnv1a64(b) == CARD[name + ".in.b"]["fnv1a64"]
    assert a.size == CARD[name + ".in.a"]["count"] and b.size == CARD[name + ".in.b"]["count"]
    c = oracle.gemm(a, b, OPS[op])
    assert c.size == CARD[name + ".out"]["count"]
    assert "%016x" % oracle.fnv1a64(c) == CARD[name + ".out"]["fnv1a64"]
    fast = oracle.gemm_rows(a, b, OPS[op])
    assert fast.tobytes() == c.tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_fixture_hashes(kind):
    assert oracle.sha16(fixtures.fixture(kind)) == TABLE["fixtures"][kind]["X"]
    assert oracle.sha16(fixtures.fixture(kind, seed=1)) == TABLE["heldout"][kind]["X"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane", sorted(lanes.LANES))
def test_verify_table_train_cell(lane, kind):
    X = fixtures.fixture(kind)
    parts = lanes.LANES[lane](lanes.OracleImpl(oracle), X)
    assert oracle.train_hash(parts) == TABLE["cells"]["%s/%s" % (lane, kind)]["train"]


def test_denormal_fixture_exercises_the_flush():
    """The `denormal` and `denormal_ftz` cells agree in the table because the
    profile flushes its operands; the fixtures themselves differ."""
    d, z = fixtures.fixture("denormal"), fixtures.fixture("denormal_ftz")
    assert d.tobytes() != z.tobytes()
    a = oracle.gemm(np.ascontiguousarray(d[:64].T), d[:64])
    b = oracle.gemm(np.ascontiguousarray(z[:64].T), z[:64])
    assert a.tobytes() == b.tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane", sorted(lanes.BATCH_LANES))
def test_verify_table_batch_cell(lane, kind):
    """The table's `batch` column: the product's rows alone, split 1 / 7 / rest and whole give the same bytes (the
    leaf size may not read m), and the whole-batch rows hash to the reference's cell."""
    Xh = fixtures.fixture(kind, seed=1)
    digest, calls = lanes.BATCH_LANES[lane](lanes.OracleImpl(oracle), Xh)
    assert digest == TABLE["cells"]["%s/%s" % (lane, kind)]["batch"]
    for fn, rows in calls:
        whole = np.asarray(fn(rows))
        assert np.asarray(fn(rows[3:4])).tobytes() == whole[3:4].tobytes()
        parts = [np.asarray(fn(rows[a:b])) for a, b in ((0, 1), (1, 8), (8, rows.shape[0]))]
        assert np.concatenate(parts, axis=0).tobytes() == whole.tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_lowbit_conversions_batch_cell(kind):
    """The `batch` column of lowbit-conversions: held-out rows packed and materialised; a row packed alone gives the
    bytes it gives inside the block (the int8 exponent belongs to the row)."""
    digest, fn, rows = lanes.lowbit_conversions_batch(lanes.OracleImpl(oracle), fixtures.fixture(kind, seed=1), lanes.LOWBIT_COLS)
    assert digest == TABLE["cells"]["lowbit-conversions/%s" % kind]["batch"]
    whole, alone = fn(rows), fn(rows[5:6])
    for w, a in zip(whole, alone):
        assert np.asarray(a).tobytes() == np.asarray(w)[5:6].tobytes()

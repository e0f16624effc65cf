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

"""The decoder-block oracle against the verify table's transformer cells, and
its own structural properties (decode equals prefill, batch rows independent)."""
import json
import math
import os

import numpy as np
import pytest

import decoder_ref
import fixtures
import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TABLE = json.load(open(os.path.join(GOLDEN, "verify_table_cells.json")))


def _materialise(w, fmt):
    out = dict(w)
    for name, a in w.items():
        if a.ndim != 2:
            continue
        if fmt == "bfloat16":
            out[name] = oracle.from_bf16(oracle.to_bf16(a))
        elif fmt == "int8":
            out[name] = oracle.dequantize_int8(*oracle.quantize_int8(a))
    return out


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_infer_cell(lane, fmt, kind):
    """forward of the held-out (2, 16, 32) slab hashes to the table's `infer` cell (tools/identity_break.py:3639-3653, :3729-3737)."""
    w, dims = decoder_ref.transformer_lane_weights()
    cfg = oracle.block_cfg(dims["d_model"], dims["n_heads"], dims["n_kv_heads"], dims["head_dim"], dims["inter"],
                           window=decoder_ref.lane_window(lane))
    x = decoder_ref.seq(fixtures.fixture(kind, seed=1), 2, 16, dims["d_model"])
    slots = decoder_ref.block_slots(_materialise(w, fmt))
    y = oracle.block_forward(cfg, slots, x)
    assert oracle.sha16(y) == TABLE["cells"]["%s/%s" % (lane, kind)]["infer"]
    # the `stepfull` column: the same forward against a zero state stepped one position at a time
    state = oracle.KVState(2, dims["n_kv_heads"], 16, dims["head_dim"])
    steps = [oracle.block_forward(cfg, slots, x[:, t:t + 1].copy(), state) for t in range(16)]
    assert np.concatenate(steps, axis=1).tobytes() == y.tobytes()
    assert decoder_ref.stepfull_cell_hash(y) == TABLE["cells"]["%s/%s" % (lane, kind)]["stepfull"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_batch_cell(lane, fmt, kind):
    """The `batch` column: forward of the held-out (8, 16, 32) slab; a sequence alone and a prefix reproduce the whole
    batch's bytes, and the whole-batch rows hash to the reference's cell (tools/identity_break.py:9591-9604)."""
    w, dims = decoder_ref.transformer_lane_weights()
    cfg = oracle.block_cfg(dims["d_model"], dims["n_heads"], dims["n_kv_heads"], dims["head_dim"], dims["inter"],
                           window=decoder_ref.lane_window(lane))
    slots = decoder_ref.block_slots(_materialise(w, fmt))
    x = decoder_ref.seq(fixtures.fixture(kind, seed=1), 8, 16, dims["d_model"])
    y = oracle.block_forward(cfg, slots, x)
    assert decoder_ref.batch_cell_hash_block(y) == TABLE["cells"]["%s/%s" % (lane, kind)]["batch"]
    assert oracle.block_forward(cfg, slots, x[2:3].copy()).tobytes() == y[2:3].tobytes()
    assert oracle.block_forward(cfg, slots, x[:, :7].copy()).tobytes() == np.ascontiguousarray(y[:, :7]).tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_ragged_cell(lane, fmt, kind):
    """The `ragged` column: every row at its own length (up to 300 positions, past the 128-step leaf of the products
    inside), padding exactly +0.0; the padded outputs hash to the reference's cell."""
    w, dims = decoder_ref.transformer_lane_weights()
    cfg = oracle.block_cfg(dims["d_model"], dims["n_heads"], dims["n_kv_heads"], dims["head_dim"], dims["inter"],
                           window=decoder_ref.lane_window(lane))
    slots = decoder_ref.block_slots(_materialise(w, fmt))
    outs = []
    for x, lens in decoder_ref.ragged_inputs(fixtures.fixture(kind, seed=1), dims["d_model"]):
        y = np.zeros_like(x)
        for i, n in enumerate(lens):
            y[i, :n] = oracle.block_forward(cfg, slots, np.ascontiguousarray(x[i:i + 1, :n]))[0]
        outs.append((x, lens, y))
    assert decoder_ref.ragged_cell_hash(outs) == TABLE["cells"]["%s/%s" % (lane, kind)]["ragged"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_batchscale_cell(lane, fmt, kind):
    """The `batchscale` column: 1024 sequences in one call and a 1024-position call whose key axis crosses seven
    128-step boundaries; sub-batches and prefixes give the whole call's bytes, which hash to the reference's cell."""
    w, dims = decoder_ref.transformer_lane_weights()
    cfg = oracle.block_cfg(dims["d_model"], dims["n_heads"], dims["n_kv_heads"], dims["head_dim"], dims["inter"],
                           window=decoder_ref.lane_window(lane))
    slots = decoder_ref.block_slots(_materialise(w, fmt))
    x, xl = decoder_ref.batchscale_inputs(fixtures.fixture(kind, seed=1), dims["d_model"])
    y, yl = oracle.block_forward(cfg, slots, x), oracle.block_forward(cfg, slots, xl)
    assert decoder_ref.batchscale_cell_hash(y, yl) == TABLE["cells"]["%s/%s" % (lane, kind)]["batchscale"]
    assert oracle.block_forward(cfg, slots, np.ascontiguousarray(x[503:520])).tobytes() == y[503:520].tobytes()
    for p in (129, 257):
        assert oracle.block_forward(cfg, slots, np.ascontiguousarray(xl[:, :p])).tobytes() == np.ascontiguousarray(yl[:, :p]).tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_transformer_decode_session_cells(kind):
    """The `transformer-decode-session` lane: `train` = the 16 stepped positions, the chunked prefill, the resident
    caches and the refusal flags; `stepfull` = the forward under the session's label; `infer` = the transformer lane's."""
    w, dims = decoder_ref.transformer_lane_weights()
    cfg = oracle.block_cfg(dims["d_model"], dims["n_heads"], dims["n_kv_heads"], dims["head_dim"], dims["inter"])
    slots = decoder_ref.block_slots(_materialise(w, "float32"))
    X, dm = fixtures.fixture(kind), dims["d_model"]
    x = decoder_ref.seq(X, 2, 16, dm)
    state = oracle.KVState(2, dims["n_kv_heads"], 32, dims["head_dim"])
    steps = [oracle.block_forward(cfg, slots, x[:, t:t + 1].copy(), state) for t in range(16)]
    prefill = oracle.block_forward(cfg, slots, decoder_ref.seq(X, 2, 16, dm, skip=1024), oracle.KVState(2, dims["n_kv_heads"], 32, dims["head_dim"]))
    parts = decoder_ref.decode_session_parts(steps, prefill, decoder_ref.packed_cache(state.k, 16), decoder_ref.packed_cache(state.v, 16))
    cell = TABLE["cells"]["transformer-decode-session/%s" % kind]
    assert oracle.train_hash(parts) == cell["train"]
    y = oracle.block_forward(cfg, slots, decoder_ref.seq(fixtures.fixture(kind, seed=1), 2, 16, dm))
    assert decoder_ref.stepfull_cell_hash(y, "decode_session step") == cell["stepfull"]
    assert oracle.sha16(y) == cell["infer"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_embedding_lane_infer_and_batch_cells(kind):
    """The gather Y = ftz(W[id]) on the verify table's `embedding` lane: 512 held-out ids (`infer`), and 64 ids whose
    rows alone give the whole call's bytes (`batch`)."""
    w, ids, ids64 = decoder_ref.embedding_lane(fixtures.fixture(kind, seed=1))
    y = oracle.embedding(w, ids.reshape(1, -1)).reshape(len(ids), -1)
    assert oracle.sha16(y) == TABLE["cells"]["embedding/%s" % kind]["infer"]
    y64 = oracle.embedding(w, ids64.reshape(1, -1)).reshape(64, -1)
    assert decoder_ref.rows_cell_hash("forward", y64) == TABLE["cells"]["embedding/%s" % kind]["batch"]
    assert oracle.embedding(w, ids64[5:6].reshape(1, 1)).reshape(1, -1).tobytes() == y64[5:6].tobytes()


def test_portable_math_is_close_to_libm_and_exact_at_anchors():
    assert oracle.math("powf", 10000.0, 0.0) == 1.0
    assert oracle.math("rsqrtf", 16.0) == 0.25 and oracle.math("rsqrtf", 64.0) == 0.125
    assert oracle.math("sqrtf", 2.0) == np.float32(math.sqrt(2.0))  # correctly rounded
    rng = np.random.default_rng(0)
    for x in rng.uniform(-20, 20, 200).astype(np.float32):
        x = float(x)
        assert abs(float(oracle.math("expf", x)) - math.exp(x)) <= 1e-6 * math.exp(x)
        assert abs(float(oracle.math("tanhf", x)) - math.tanh(x)) <= 1e-6
        y = float(np.float32(x / 5))
        assert abs(float(oracle.math("erff", y)) - math.erf(y)) <= 1e-6
    for x in rng.uniform(0, 8000, 200).astype(np.float32):
        x = float(x)
        assert abs(float(oracle.math("cosf", x)) - math.cos(x)) <= 1e-6
        assert abs(float(oracle.math("sinf", x)) - math.sin(x)) <= 1e-6
    assert oracle.math("fmaxf", -0.0, 0.0).view(np.uint32) == 0 and oracle.math("fmaxf", 0.0, -0.0).view(np.uint32) == 0


@pytest.mark.parametrize("opts", [dict(), dict(norm="layernorm", norm_bias=True, mlp="gelu", mlp_bias=True, qkv_bias=True, o_bias=True, rope=False),
                                  dict(mlp="gelu_tanh", n_kv_heads=4)])
def test_decode_equals_prefill_and_rows_are_independent(opts):
    rng = np.random.default_rng(1)
    dm, nh, hd, it = 48, 4, 12, 300  # k = 300 in the down projection: three leaves, one carry
    nkv = opts.pop("n_kv_heads", 2)
    cfg = oracle.block_cfg(dm, nh, nkv, hd, it, **opts)
    gated = cfg.mlp_kind in (0, 4, 5)
    w = {"norm1": 1 + rng.standard_normal(dm) * 0.1, "norm2": 1 + rng.standard_normal(dm) * 0.1,
         "q": rng.standard_normal((nh * hd, dm)) * 0.2, "k": rng.standard_normal((nkv * hd, dm)) * 0.2,
         "v": rng.standard_normal((nkv * hd, dm)) * 0.2, "o": rng.standard_normal((dm, nh * hd)) * 0.2,
         "up": rng.standard_normal((it, dm)) * 0.2, "down": rng.standard_normal((dm, it)) * 0.2}
    if gated:
        w["gate"] = rng.standard_normal((it, dm)) * 0.2
    for b_, width in (("norm1_b", dm), ("norm2_b", dm), ("q_b", nh * hd), ("k_b", nkv * hd), ("v_b", nkv * hd), ("o_b", dm),
                      ("up_b", it), ("down_b", dm), ("gate_b", it)):
        w[b_] = rng.standard_normal(width) * 0.1
    w = {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}
    x = rng.standard_normal((3, 9, dm)).astype(np.float32)
    whole = oracle.block_forward(cfg, w, x)
    state = oracle.KVState(3, nkv, 9, hd)
    first = oracle.block_forward(cfg, w, x[:, :5].copy(), state)
    rest = [oracle.block_forward(cfg, w, x[:, t:t + 1].copy(), state) for t in range(5, 9)]
    assert np.concatenate([first] + rest, axis=1).tobytes() == whole.tobytes()
    alone = oracle.block_forward(cfg, w, x[1:2].copy())
    assert alone.tobytes() == whole[1:2].tobytes()


def test_argmax_ties_go_to_the_lowest_id():
    logits = np.array([[1.0, 3.0, 3.0, -1.0], [0.0, -0.0, 0.0, 0.0], [np.nan, 2.0, 1.0, 2.0]], dtype=np.float32)
    assert oracle.argmax(logits).tolist() == [1, 0, 0]


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_hf_causal_lm_infer_cell(kind):
    """The verify table's `hf-causal-lm` lane, `infer` column: the logits of the Llama-shaped synthetic checkpoint
    (embedding, two rotary GQA blocks, final RMSNorm, untied head) on 4 x 12 ids cut from the held-out fixture's
    bytes. Pins the whole decoder, embedding to head, on the reference's own hash."""
    ids = decoder_ref.fixture_ids(fixtures.fixture(kind, seed=1), 4, 12, decoder_ref.LlamaFixtureConfig.vocab)
    lm = decoder_ref.OracleLM(decoder_ref.LlamaFixtureConfig, decoder_ref.llama_fixture_weights())
    logits = lm.forward(ids)
    assert oracle.sha16(logits) == TABLE["cells"]["hf-causal-lm/%s" % kind]["infer"]
    # the `batch` column: the same logits hashed row by row and as the full-length prefix answer; a row alone and a
    # prefix give the whole batch's bytes
    assert decoder_ref.batch_cell_hash(logits) == TABLE["cells"]["hf-causal-lm/%s" % kind]["batch"]
    assert lm.forward(ids[1:2]).tobytes() == logits[1:2].tobytes()
    assert lm.forward(ids[:, :7]).tobytes() == np.ascontiguousarray(logits[:, :7]).tobytes()


def test_masked_score_is_the_fill_when_operands_are_small():
    """The prefill score kernel writes -FLT_MAX for a tile no query can see without forming its dot products when
    every operand word is finite and below 2^40: a dot of up to 128 such products stays under 2^88, half an ulp of
    FLT_MAX is 2^103, so score + (-FLT_MAX) rounds back to -FLT_MAX. Checked here at the bound and just above it."""
    fill = np.frombuffer(np.uint32(0xFF7FFFFF).tobytes(), dtype=np.float32)[0]
    for mag in (0.0, 1.0, 2.0 ** 87, 2.0 ** 88, 2.0 ** 102):
        for sign in (1.0, -1.0):
            assert np.float32(np.float32(sign * mag) + fill) == fill
    assert np.float32(np.float32(2.0 ** 104) + fill) != fill  # a score this large does move the sum: the kernel computes such tiles
    # the largest dot the shortcut admits: 128 products of two words just below 2^40
    x = np.float32(np.nextafter(np.float32(2.0 ** 40), np.float32(0)))
    assert float(x) * float(x) * 128 < 2.0 ** 88


def test_rotary_table_options_default_record_is_the_frozen_table():
    """The option record at its defaults (no scaling, rope_dim = head_dim) is the v1 table bit for bit; a linear factor
    divides every inverse frequency once, so the table at position p is not the default table anywhere but p = 0."""
    cos0, sin0 = oracle.rope_table(3, 20, 16, 10000.0)
    cos1, sin1 = oracle.rope_table_opts(3, 20, 16, 10000.0, None)
    assert cos0.tobytes() == cos1.tobytes() and sin0.tobytes() == sin1.tobytes()
    cos2, sin2 = oracle.rope_table_opts(0, 20, 16, 10000.0, {"rope_type": "linear", "factor": 4.0})
    base_c, base_s = oracle.rope_table(0, 20, 16, 10000.0)
    assert cos2[0].tobytes() == base_c[0].tobytes() and cos2[4, 0] == base_c[1, 0] and not np.array_equal(cos2[1], base_c[1])
    cos3, _ = oracle.rope_table_opts(0, 20, 16, 10000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                          "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    assert np.isfinite(cos3).all() and cos3[:, 0].tobytes() == base_c[:, 0].tobytes()  # the highest frequency keeps its wavelength
    assert not np.array_equal(cos3[:, 7], base_c[:, 7])  # the lowest one is slowed by the factor
    cos4, _ = oracle.rope_table_opts(0, 20, 8, 10000.0, None)  # a partial rotary's table is the table of a narrower head
    assert cos4.tobytes() == oracle.rope_table(0, 20, 8, 10000.0)[0].tobytes()

"""GPU parity for the decoder path: the block's seams and the CausalLM against
the CPU oracle, bit for bit, and against the verify table's transformer cells."""
import ctypes
import json
import os

import numpy as np
import pytest

import decoder_ref
import fixtures
import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native, lowbit  # noqa: E402
from mojolearn_b200.models import CausalLM, CausalLMConfig  # noqa: E402
from mojolearn_b200.transformer import TransformerBlock  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TABLE = json.load(open(os.path.join(GOLDEN, "verify_table_cells.json")))


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_infer_cell_on_gpu(lane, fmt, kind):
    w, dims = decoder_ref.transformer_lane_weights()
    packed = lowbit.pack(w, fmt) if fmt != "float32" else w
    blk = TransformerBlock(packed, n_heads=dims["n_heads"], n_kv_heads=dims["n_kv_heads"], window=decoder_ref.lane_window(lane))
    assert blk.weight_format == fmt
    x = decoder_ref.seq(fixtures.fixture(kind, seed=1), 2, 16, dims["d_model"])
    y = blk.forward(x)
    assert oracle.sha16(y) == TABLE["cells"]["%s/%s" % (lane, kind)]["infer"]
    # the `stepfull` column: allocate_state + one step per position reproduces the forward, which hashes to the cell
    state = blk.allocate_state(2, 16)
    steps = [blk.step(np.ascontiguousarray(x[:, t:t + 1]), state) for t in range(16)]
    assert np.concatenate(steps, axis=1).tobytes() == y.tobytes()
    assert decoder_ref.stepfull_cell_hash(y) == TABLE["cells"]["%s/%s" % (lane, kind)]["stepfull"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_batch_cell_on_gpu(lane, fmt, kind):
    """The table's `batch` column on the CUDA path: forward of the held-out (8, 16, 32) slab; every sequence alone,
    the split 1 / 7 and the prefixes 1, 7, 15 reproduce the whole batch's bytes, which hash to the reference's cell."""
    w, dims = decoder_ref.transformer_lane_weights()
    packed = lowbit.pack(w, fmt) if fmt != "float32" else w
    blk = TransformerBlock(packed, n_heads=dims["n_heads"], n_kv_heads=dims["n_kv_heads"], window=decoder_ref.lane_window(lane))
    x = decoder_ref.seq(fixtures.fixture(kind, seed=1), 8, 16, dims["d_model"])
    y = blk.forward(x)
    assert decoder_ref.batch_cell_hash_block(y) == TABLE["cells"]["%s/%s" % (lane, kind)]["batch"]
    for a, b in ((0, 1), (1, 8), (3, 4)):
        assert blk.forward(np.ascontiguousarray(x[a:b])).tobytes() == y[a:b].tobytes()
    for p in (1, 7, 15):
        assert blk.forward(np.ascontiguousarray(x[:, :p])).tobytes() == np.ascontiguousarray(y[:, :p]).tobytes()


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_ragged_cell_on_gpu(lane, fmt, kind):
    """The table's `ragged` column on the CUDA path: forward(x, lengths=...) with NaN junk in the padding; real positions
    equal the row alone, padding is exactly +0.0, and the padded outputs hash to the reference's cell."""
    w, dims = decoder_ref.transformer_lane_weights()
    packed = lowbit.pack(w, fmt) if fmt != "float32" else w
    blk = TransformerBlock(packed, n_heads=dims["n_heads"], n_kv_heads=dims["n_kv_heads"], window=decoder_ref.lane_window(lane))
    outs = []
    for x, lens in decoder_ref.ragged_inputs(fixtures.fixture(kind, seed=1), dims["d_model"]):
        y = blk.forward(x, lengths=lens)
        assert not np.isnan(y).any()
        for i, n in enumerate(lens):
            assert y[i, n:].tobytes() == bytes(y[i, n:].nbytes)
        i = 2
        assert blk.forward(np.ascontiguousarray(x[i:i + 1, :lens[i]])).tobytes() == np.ascontiguousarray(y[i:i + 1, :lens[i]]).tobytes()
        outs.append((x, lens, y))
    assert decoder_ref.ragged_cell_hash(outs) == TABLE["cells"]["%s/%s" % (lane, kind)]["ragged"]
    with pytest.raises(ValueError):
        blk.forward(outs[0][0], state=blk.allocate_state(8, 16), lengths=outs[0][1])


@pytest.mark.parametrize("kind", fixtures.KINDS)
@pytest.mark.parametrize("lane,fmt", decoder_ref.LANE_FORMATS)
def test_transformer_batchscale_cell_on_gpu(lane, fmt, kind):
    """The table's `batchscale` column on the CUDA path: the 1024-row call against sub-batches of 1, 17, 64 and 256 rows
    at three offsets, the 1024-position call against prefixes around the 64 / 128 / 256 / 512 boundaries."""
    w, dims = decoder_ref.transformer_lane_weights()
    packed = lowbit.pack(w, fmt) if fmt != "float32" else w
    blk = TransformerBlock(packed, n_heads=dims["n_heads"], n_kv_heads=dims["n_kv_heads"], window=decoder_ref.lane_window(lane))
    x, xl = decoder_ref.batchscale_inputs(fixtures.fixture(kind, seed=1), dims["d_model"])
    y, yl = blk.forward(x), blk.forward(xl)
    assert decoder_ref.batchscale_cell_hash(y, yl) == TABLE["cells"]["%s/%s" % (lane, kind)]["batchscale"]
    for b in (1, 17, 64, 256):
        for a in sorted({0, (1024 - b) // 2, 1024 - b}):
            assert blk.forward(np.ascontiguousarray(x[a:a + b])).tobytes() == y[a:a + b].tobytes(), (b, a)
    for p in decoder_ref.SCALE_PREFIXES:
        assert blk.forward(np.ascontiguousarray(xl[:, :p])).tobytes() == np.ascontiguousarray(yl[:, :p]).tobytes(), p


OPTION_SETS = [
    dict(),
    dict(norm="layernorm", norm_bias=True, mlp="gelu", mlp_bias=True, qkv_bias=True, o_bias=True, positions="learned"),
    dict(mlp="gelu_tanh", n_kv_heads=4, norm="rmsnorm_offset"),
    dict(mlp="geglu", window=5),
    # the option record of transformer/block_options.mojo:40-70 of the reference: q/k norms, score soft cap, partial
    # rotary, linear and llama3 frequency scaling (their spellings are the reference oracle's; no committed hash pins them)
    dict(qk_norm=True, attn_softcap=30.0),
    dict(qk_norm=True, norm="rmsnorm_offset", rope_dim=8, rope_theta=500000.0),
    dict(rope_scaling={"rope_type": "linear", "factor": 4.0}, mlp="silu"),
    dict(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 16}, attn_softcap=2.5, qkv_bias=True),
]


@pytest.mark.parametrize("opts", OPTION_SETS)
def test_causal_lm_matches_the_oracle_and_decode_equals_prefill(opts):
    opts = dict(opts)
    cfg = CausalLMConfig(vocab=97, d_model=48, n_layers=2, n_heads=4, n_kv_heads=opts.pop("n_kv_heads", 2), head_dim=12,
                         intermediate=300, max_positions=64, **opts)
    w = decoder_ref.random_lm_weights(cfg, seed=3, scale=0.2)
    ref = decoder_ref.OracleLM(cfg, w)
    lm = CausalLM(cfg, w)
    ids = np.random.default_rng(0).integers(0, cfg.vocab, (3, 9)).astype(np.int32)
    want = ref.forward(ids)
    got = lm.forward(ids)
    assert got.tobytes() == want.tobytes()
    state = lm.allocate_state(3, 9)
    first = lm.forward(ids[:, :5], state)
    rest = [lm.step(ids[:, t], state) for t in range(5, 9)]
    assert np.concatenate([first] + [r[:, None, :] for r in rest], axis=1).tobytes() == want.tobytes()
    seq, logits = lm.generate(ids[:, :4], 6, return_logits=True)  # steps 2.. replay the captured graph
    rseq, rlogits = ref.generate(ids[:, :4], 6)
    assert seq.tolist() == rseq.tolist() and logits.tobytes() == rlogits.tobytes()
    seq2, logits2 = lm.generate(ids[:, :4], 6, return_logits=True, graph=False)
    assert seq2.tolist() == rseq.tolist() and logits2.tobytes() == rlogits.tobytes()
    with pytest.raises(ValueError):
        lm.forward(np.full((1, 2), cfg.vocab, np.int32))
    # the reference's other doors on the same model: a stream reads the same continuation, a reset state is a fresh one
    stream = lm.stream(ids[:, :4], 6)
    got = np.concatenate([stream.read(4), stream.read(4), stream.read(4)], axis=1)
    assert got.tolist() == rseq[:, 4:].tolist() and stream.read(1).shape == (3, 0)
    state = lm.reset_state(state)
    assert state.positions == 0 and lm.forward(ids, state).tobytes() == want.tobytes()


def test_block_option_refusals_and_weight_format():
    cfg = CausalLMConfig(vocab=97, d_model=48, n_layers=1, n_heads=4, n_kv_heads=2, head_dim=12, intermediate=64, max_positions=64)
    w = decoder_ref.random_lm_weights(cfg, seed=4, scale=0.2)
    bw = {k[len("model.layers.0."):].replace("self_attn.", "").replace("mlp.", ""): v for k, v in w.items() if k.startswith("model.layers.0.")}
    with pytest.raises(ValueError, match="rope_dim"):
        TransformerBlock(bw, n_heads=4, n_kv_heads=2, rope_dim=7)
    with pytest.raises(ValueError, match="rope_scaling"):
        TransformerBlock(bw, n_heads=4, n_kv_heads=2, rope_scaling={"rope_type": "yarn", "factor": 2.0})
    with pytest.raises(ValueError, match="q_norm.weight"):
        TransformerBlock(bw, n_heads=4, n_kv_heads=2, qk_norm=True)
    with pytest.raises(ValueError, match="attn_softcap"):
        TransformerBlock(bw, n_heads=4, n_kv_heads=2, attn_softcap=-1.0)
    with pytest.raises(ValueError, match="numeric_profile"):
        TransformerBlock(bw, n_heads=4, n_kv_heads=2, numeric_profile="int15")
    with pytest.raises(ValueError, match="weight_format"):
        CausalLM(cfg, w, weight_format="fp8")
    ids = np.random.default_rng(1).integers(0, cfg.vocab, (2, 7)).astype(np.int32)
    # weight_format packs the float32 projections on the way in: the logits are the oracle's on the materialised weights
    for fmt in ("bfloat16", "int8"):
        lm = CausalLM(cfg, w, weight_format=fmt, max_positions=32)
        assert lm.config.max_positions == 32 and lm.blocks[0].weight_format == fmt
        mat = {k: (lowbit.materialize_one(lowbit.pack_one(v, fmt)) if (v.ndim == 2 and "embed" not in k) else v) for k, v in w.items()}
        assert lm.forward(ids).tobytes() == decoder_ref.OracleLM(cfg, mat).forward(ids).tobytes()
        with pytest.raises(ValueError, match="max_positions"):
            lm.forward(np.zeros((1, 33), np.int32))
    names = CausalLM(cfg, w).parameters()
    assert "model.layers.0.q_proj.weight" in names or "model.layers.0.input_layernorm.weight" in names


def test_block_subnormal_forcing_inputs():
    w, dims = decoder_ref.transformer_lane_weights()
    blk = TransformerBlock(w, n_heads=2, n_kv_heads=1)
    cfg = oracle.block_cfg(32, 2, 1, 16, 64)
    x = decoder_ref.seq(fixtures.fixture("base", seed=1), 2, 16, 32) * np.float32(2.0 ** -70)
    x[0, 3, :5] = np.float32(1e-41)
    want = oracle.block_forward(cfg, decoder_ref.block_slots(w), x)
    assert blk.forward(x).tobytes() == want.tobytes()


def test_prefill_attention_extreme_operands():
    """A prompt longer than two score tiles with queries and keys near 2^48 (a tile no query can see must then form
    its dot products: they are large enough to move the masked sum) and values near 2^-100 (the value chain must
    take the flushed step), and the same block with ordinary weights for the tiles written without dot products."""
    w, dims = decoder_ref.transformer_lane_weights()
    cfg = oracle.block_cfg(32, 2, 1, 16, 64)
    x = decoder_ref.seq(np.asarray(decoder_ref.lcg_floats(2 * 130 * 32, 5, -1.0, 1.0), dtype=np.float32), 2, 130, 32)
    for qk, v in ((np.float32(2.0 ** 48), np.float32(2.0 ** -100)), (np.float32(1.0), np.float32(1.0)),
                  (np.float32(2.0 ** 54), np.float32(1.0))):
        w2 = dict(w)
        w2["q_proj.weight"] = w["q_proj.weight"] * qk
        w2["k_proj.weight"] = w["k_proj.weight"] * qk
        w2["v_proj.weight"] = w["v_proj.weight"] * v
        want = oracle.block_forward(cfg, decoder_ref.block_slots(w2), x)
        got = TransformerBlock(w2, n_heads=2, n_kv_heads=1).forward(x)
        assert got.tobytes() == want.tobytes(), (float(qk), float(v))


def test_config4_shape_reduced_length():
    """The GPT-2-small style benchmark architecture (12 layers would only repeat the block: 2 here), d_model 768, 12 heads,
    MLP 3072 GELU, LayerNorm, learned positions, vocab 50304, batch 8: prompt 24 tokens then 4 greedy steps."""
    cfg = CausalLMConfig(vocab=50304, d_model=768, n_layers=2, n_heads=12, intermediate=3072, norm="layernorm", norm_bias=True,
                         mlp="gelu", mlp_bias=True, qkv_bias=True, o_bias=True, positions="learned", max_positions=64)
    w = decoder_ref.random_lm_weights(cfg, seed=0, scale=0.02)
    ids = np.random.default_rng(0).integers(0, cfg.vocab, (8, 24)).astype(np.int32)
    seq, logits = CausalLM(cfg, w).generate(ids, 4, return_logits=True)
    rseq, rlogits = decoder_ref.OracleLM(cfg, w).generate(ids, 4)
    assert logits.tobytes() == rlogits.tobytes() and seq.tolist() == rseq.tolist()


def test_config5_shape_int8_weights_reduced():
    """The serving benchmark's layer shapes (d_model 2048, 16 heads of 128, MLP 8192, vocab 50304, INT8 weights with
    power-of-two row exponents), 1 layer, batch 4, prompt 20 then 3 steps, against the oracle on the materialised weights."""
    cfg = CausalLMConfig(vocab=50304, d_model=2048, n_layers=1, n_heads=16, intermediate=8192, max_positions=64)
    w = decoder_ref.random_lm_weights(cfg, seed=1, scale=0.02)
    packed = {k: (lowbit.pack_one(v, "int8") if (v.ndim == 2 and "embed" not in k) else v) for k, v in w.items()}
    mat = {k: lowbit.materialize_one(v) for k, v in packed.items()}
    ids = np.random.default_rng(2).integers(0, cfg.vocab, (4, 20)).astype(np.int32)
    seq, logits = CausalLM(cfg, packed).generate(ids, 3, return_logits=True)
    rseq, rlogits = decoder_ref.OracleLM(cfg, mat).generate(ids, 3)
    assert logits.tobytes() == rlogits.tobytes() and seq.tolist() == rseq.tolist()


def test_argmax_kernel_ties_nans_and_wide_rows():
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((7, 50304)).astype(np.float32)
    logits[1, 40000] = logits[1, 123] = logits[1].max() + 1.0      # a tie: the lower index wins
    logits[2, 0] = np.nan                                          # a NaN at element 0 is never displaced
    logits[3, 5:9000] = np.nan                                     # NaNs elsewhere are never candidates
    logits[4, :] = 0.0
    logits[4, 77] = -0.0                                           # signed zeros compare equal
    logits[5, :] = -np.inf
    logits[6, -1] = np.inf
    small = np.array([[1.0, 3.0, 3.0, -1.0], [0.0, -0.0, 0.0, 0.0], [np.nan, 2.0, 1.0, 2.0]], dtype=np.float32)
    for arr in (logits, small, logits[:, :1], logits[:, :1025]):
        arr = np.ascontiguousarray(arr)
        d = torch.from_numpy(arr).cuda()
        out = torch.empty(arr.shape[0], dtype=torch.int32, device="cuda")
        _native.call("b200i_argmax", 0, None, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(d.data_ptr()), arr.shape[0], arr.shape[1])
        torch.cuda.synchronize()
        assert out.cpu().numpy().tolist() == oracle.argmax(arr).tolist()


def test_norm_kernel_row_widths_and_kinds():
    """Rows staged in shared memory: vector and scalar widths, one and many rows per launch, the three kinds,
    rows that fail the admission test of the sum of squares."""
    from mojolearn_b200 import transformer
    rng = np.random.default_rng(6)
    for rows, dm in [(1, 4), (3, 37), (32, 2048), (5, 1000), (1500, 96), (2, 8192)]:
        x = rng.standard_normal((rows, dm)).astype(np.float32)
        x[0, :: 5] *= np.float32(2.0 ** -70)  # below the admission threshold: the flushed chain
        if rows > 1:
            x[1, 0] = np.float32(1e-41)
        w = rng.standard_normal(dm).astype(np.float32)
        bias = rng.standard_normal(dm).astype(np.float32)
        for name, b in (("rmsnorm", None), ("layernorm", bias), ("layernorm", None), ("rmsnorm_offset", None)):
            kind = transformer.NORM_KINDS[name]
            want = oracle.norm(x, w, b, 1e-6, name)
            got = transformer.norm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(),
                                   None if b is None else torch.from_numpy(b).cuda(), 1e-6, kind)
            assert got.cpu().numpy().tobytes() == want.tobytes(), (rows, dm, kind)


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_hf_causal_lm_infer_cell_on_gpu(kind):
    """The verify table's `hf-causal-lm` lane, `infer` column, on the CUDA path: logits of the Llama-shaped synthetic
    checkpoint on ids cut from the held-out fixture, against the reference's own hash; a prefill of 11 tokens plus
    one step (launch by launch and replayed from the graph) gives the same last-position logits."""
    c = decoder_ref.LlamaFixtureConfig
    cfg = CausalLMConfig(vocab=c.vocab, d_model=c.d_model, n_layers=c.n_layers, n_heads=c.n_heads, n_kv_heads=c.n_kv_heads,
                         head_dim=c.head_dim, intermediate=c.intermediate, norm_eps=c.norm_eps, rope_theta=c.rope_theta,
                         max_positions=c.max_positions)
    lm = CausalLM(cfg, decoder_ref.llama_fixture_weights())
    ids = decoder_ref.fixture_ids(fixtures.fixture(kind, seed=1), 4, 12, c.vocab)
    logits = lm.forward(ids)
    assert oracle.sha16(logits) == TABLE["cells"]["hf-causal-lm/%s" % kind]["infer"]
    assert decoder_ref.batch_cell_hash(logits) == TABLE["cells"]["hf-causal-lm/%s" % kind]["batch"]
    for rows in (slice(0, 1), slice(1, 2), slice(1, 4)):  # a row alone and a split reproduce the whole batch's bytes
        assert lm.forward(ids[rows]).tobytes() == logits[rows].tobytes()
    for p in (1, 7, 11):  # and so does every prefix
        assert lm.forward(ids[:, :p]).tobytes() == np.ascontiguousarray(logits[:, :p]).tobytes()
    state = lm.allocate_state(4, 12)
    lm.forward(ids[:, :11], state)
    assert lm.step(ids[:, 11], state).tobytes() == np.ascontiguousarray(logits[:, 11, :]).tobytes()
    seq = lm.generate(ids[:, :6], 6)
    assert seq.tolist() == lm.generate(ids[:, :6], 6, graph=False).tolist()


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_transformer_decode_session_cells_on_gpu(kind):
    """The `transformer-decode-session` lane on the CUDA path: a session's 16 steps and its chunked forward are the
    per-call step and forward byte for byte, its state is the per-call state, the refusals hold, and the parts hash
    to the reference's `train`, `stepfull` and `infer` cells."""
    from mojolearn_b200.transformer import TransformerDecodeSession
    w, dims = decoder_ref.transformer_lane_weights()
    blk = TransformerBlock(w, n_heads=dims["n_heads"], n_kv_heads=dims["n_kv_heads"])
    X, dm = fixtures.fixture(kind), dims["d_model"]
    x = decoder_ref.seq(X, 2, 16, dm)
    st = blk.allocate_state(2, max_tokens=32)
    with blk.decode_session(st) as sess:
        steps = [np.ascontiguousarray(sess.step(np.ascontiguousarray(x[:, t:t + 1]))) for t in range(16)]
        sess.sync_state()
        resident = (st.k_cache, st.v_cache)
    plain = blk.allocate_state(2, max_tokens=32)
    per_call = [blk.step(np.ascontiguousarray(x[:, t:t + 1]), plain) for t in range(16)]
    assert np.concatenate(steps, axis=1).tobytes() == np.concatenate(per_call, axis=1).tobytes()
    assert resident[0].tobytes() == plain.k_cache.tobytes() and resident[1].tobytes() == plain.v_cache.tobytes()
    chunk = decoder_ref.seq(X, 2, 16, dm, skip=1024)
    with blk.decode_session(blk.allocate_state(2, max_tokens=32)) as sess:
        prefill = np.ascontiguousarray(sess.forward(chunk))
    assert prefill.tobytes() == blk.forward(chunk, blk.allocate_state(2, max_tokens=32)).tobytes()
    closed = blk.decode_session(blk.allocate_state(2, max_tokens=32))
    closed.close()
    busy = blk.allocate_state(2, max_tokens=32)
    open_session = blk.decode_session(busy)
    assert type(open_session) is TransformerDecodeSession and open_session.is_open and not closed.is_open
    with pytest.raises(RuntimeError, match="session is closed"):
        closed.step(np.zeros((2, 1, dm), dtype=np.float32))
    with pytest.raises(RuntimeError, match="resident"):
        blk.decode_session(busy)
    with pytest.raises(ValueError, match="state is required"):
        blk.decode_session(None)
    with pytest.raises(ValueError, match="window"):
        blk.decode_session(blk.allocate_state(2, max_tokens=32, window=8))
    open_session.close()
    cell = TABLE["cells"]["transformer-decode-session/%s" % kind]
    assert oracle.train_hash(decoder_ref.decode_session_parts(steps, prefill, *resident)) == cell["train"]
    y = blk.forward(decoder_ref.seq(fixtures.fixture(kind, seed=1), 2, 16, dm))
    assert decoder_ref.stepfull_cell_hash(y, "decode_session step") == cell["stepfull"]
    assert oracle.sha16(y) == cell["infer"]


@pytest.mark.parametrize("kind", fixtures.KINDS)
def test_embedding_lane_infer_and_batch_cells_on_gpu(kind):
    """The `embedding` lane's forward on the CUDA path (b200i_embedding): `infer` and `batch` cells of the verify table."""
    w, ids, ids64 = decoder_ref.embedding_lane(fixtures.fixture(kind, seed=1))
    dw, status = torch.from_numpy(w).cuda(), torch.zeros(1, dtype=torch.int32, device="cuda")

    def gather(some):
        di = torch.from_numpy(np.ascontiguousarray(some)).cuda()
        y = torch.empty((len(some), w.shape[1]), dtype=torch.float32, device="cuda")
        _native.call("b200i_embedding", 0, None, ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(dw.data_ptr()),
                     ctypes.c_void_p(di.data_ptr()), len(some), w.shape[0], w.shape[1], ctypes.c_void_p(status.data_ptr()))
        return y.cpu().numpy()

    assert oracle.sha16(gather(ids)) == TABLE["cells"]["embedding/%s" % kind]["infer"]
    y64 = gather(ids64)
    assert decoder_ref.rows_cell_hash("forward", y64) == TABLE["cells"]["embedding/%s" % kind]["batch"]
    for a, b in ((0, 1), (1, 8), (8, 64)):
        assert gather(ids64[a:b]).tobytes() == y64[a:b].tobytes()
    assert int(status.item()) == 0


def test_causal_lm_load_from_a_checkpoint_directory(tmp_path):
    """`CausalLM.load` (reference python/mojolearn/models/causal_lm.py:139-150): config.json + model.safetensors of a
    Qwen3-shaped model (q/k norms, grouped heads, llama3 frequency scaling) and of a tied-embedding Llama written as
    BF16; the loaded model's logits are the oracle's on the same tensors, bit for bit."""
    import json
    from mojolearn_b200.models import config as model_config, safetensors
    hf = {"model_type": "qwen3", "vocab_size": 97, "hidden_size": 48, "num_hidden_layers": 2, "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 12, "intermediate_size": 80, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
          "max_position_embeddings": 64, "hidden_act": "silu",
          "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                           "original_max_position_embeddings": 16}}
    plan = model_config.plan_for(hf)
    w = decoder_ref.random_lm_weights(plan, seed=11, scale=0.2)
    os.makedirs(tmp_path / "qwen3")
    json.dump(hf, open(tmp_path / "qwen3" / "config.json", "w"))
    safetensors.write_file(tmp_path / "qwen3" / "model.safetensors", w)
    lm = CausalLM.load(tmp_path / "qwen3")
    ids = np.random.default_rng(3).integers(0, 97, (2, 9)).astype(np.int32)
    assert lm.forward(ids).tobytes() == decoder_ref.OracleLM(plan, w).forward(ids).tobytes()
    # a tied head and BF16 storage: widened exactly, or kept as bits when asked for bfloat16 weights
    hf2 = dict(hf, model_type="llama", tie_word_embeddings=True)
    hf2.pop("rope_scaling")
    plan2 = model_config.plan_for(hf2)
    w2 = decoder_ref.random_lm_weights(plan2, seed=12, scale=0.2)
    w2.pop("lm_head.weight")
    as_bf16 = {k: oracle.to_bf16(v.reshape(1, -1) if v.ndim == 1 else v).reshape(v.shape) for k, v in w2.items()}
    os.makedirs(tmp_path / "llama")
    json.dump(hf2, open(tmp_path / "llama" / "config.json", "w"))
    safetensors.write_file(tmp_path / "llama" / "model.safetensors", as_bf16)
    wide = {k: oracle.from_bf16(v.reshape(1, -1) if v.ndim == 1 else v).reshape(v.shape) for k, v in as_bf16.items()}
    wide["lm_head.weight"] = wide["model.embed_tokens.weight"]
    want = decoder_ref.OracleLM(plan2, wide).forward(ids)
    assert CausalLM.load(tmp_path / "llama").forward(ids).tobytes() == want.tobytes()
    assert CausalLM.load(tmp_path / "llama", weight_format="bfloat16").forward(ids).tobytes() == want.tobytes()
    os.remove(tmp_path / "llama" / "model.safetensors")
    with pytest.raises(FileNotFoundError):
        CausalLM.load(tmp_path / "llama")

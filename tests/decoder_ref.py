"""The CPU-oracle composition of a decoder LM, used by the tests as the checker
for mojolearn_b200.models.CausalLM: embedding gather, (learned positions,)
blocks, final norm, head product, greedy argmax."""
import hashlib

import numpy as np

import oracle

BLOCK_NAMES = {"norm1": "input_layernorm.weight", "norm1_b": "input_layernorm.bias", "q": "self_attn.q_proj.weight",
               "q_b": "self_attn.q_proj.bias", "k": "self_attn.k_proj.weight", "k_b": "self_attn.k_proj.bias",
               "v": "self_attn.v_proj.weight", "v_b": "self_attn.v_proj.bias", "o": "self_attn.o_proj.weight",
               "o_b": "self_attn.o_proj.bias", "norm2": "post_attention_layernorm.weight",
               "norm2_b": "post_attention_layernorm.bias", "gate": "mlp.gate_proj.weight", "gate_b": "mlp.gate_proj.bias",
               "up": "mlp.up_proj.weight", "up_b": "mlp.up_proj.bias", "down": "mlp.down_proj.weight",
               "down_b": "mlp.down_proj.bias", "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight"}


def hashed_uniform(n, seed):
    """The verify harness's counter-mode sha256 stream (tools/identity_break.py:1415-1431 of the reference)."""
    ctr = np.arange(n, dtype=np.uint64)
    dig = hashlib.sha256(ctr.tobytes() + str(seed).encode()).digest()
    chunks, blk, have = [], 0, 0
    while have < n * 4:
        h = hashlib.sha256(dig + blk.to_bytes(8, "little")).digest()
        chunks.append(h)
        have += len(h)
        blk += 1
    u32 = np.frombuffer(b"".join(chunks)[: n * 4], dtype=np.uint32)
    return (u32.astype(np.float64) / 2 ** 32).astype(np.float32)


def hashed_weight(shape, seed, lo, hi):
    """tools/identity_break.py:3022-3027."""
    n = int(np.prod(shape))
    u = hashed_uniform(n, seed)
    return np.ascontiguousarray((u * np.float32(hi - lo) + np.float32(lo)).astype(np.float32).reshape(shape))


def transformer_lane_weights():
    """The nine weights of the `transformer` lane (tools/identity_break.py:3639-3653)."""
    dm, nh, nkv, hd, it = 32, 2, 1, 16, 64
    shapes = {"input_layernorm.weight": (dm,), "post_attention_layernorm.weight": (dm,), "q_proj.weight": (nh * hd, dm),
              "k_proj.weight": (nkv * hd, dm), "v_proj.weight": (nkv * hd, dm), "o_proj.weight": (dm, nh * hd),
              "gate_proj.weight": (it, dm), "up_proj.weight": (it, dm), "down_proj.weight": (dm, it)}
    near_one = ("input_layernorm.weight", "post_attention_layernorm.weight")
    w = {}
    for name, shp in shapes.items():
        if name in near_one:
            w[name] = (np.float32(1.0) + hashed_weight(shp, "transformer:near_one:" + name, -0.125, 0.125)).astype(np.float32)
        else:
            w[name] = hashed_weight(shp, "transformer:" + name, -0.125, 0.125)
    return w, dict(d_model=dm, n_heads=nh, n_kv_heads=nkv, head_dim=hd, inter=it)


def seq(X, b, l, dm, skip=0):
    flat = np.ascontiguousarray(X).reshape(-1)
    return np.ascontiguousarray(flat[skip: skip + b * l * dm].reshape(b, l, dm)).astype(np.float32)


def block_slots(weights, prefix=""):
    """HuggingFace-named block weights -> the oracle's slot dict (materialised float32)."""
    out = {}
    for slot, name in BLOCK_NAMES.items():
        for key in (prefix + name, prefix + name.replace("self_attn.", "").replace("mlp.", "")):
            if key in weights:
                out[slot] = np.asarray(weights[key], dtype=np.float32)
    return out


def random_lm_weights(cfg, seed, scale=0.02):
    """HuggingFace-named float32 weights for a CausalLMConfig, N(0, scale), norm weights near one."""
    rng = np.random.default_rng(seed)

    def mat(*shape):
        return (rng.standard_normal(shape) * scale).astype(np.float32)

    hd, nh, nkv, dm, it = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_model, cfg.intermediate
    w = {"model.embed_tokens.weight": mat(cfg.vocab, dm), "model.norm.weight": (1 + mat(dm)).astype(np.float32),
         "lm_head.weight": mat(cfg.vocab, dm)}
    if cfg.norm_bias:
        w["model.norm.bias"] = mat(dm)
    if cfg.positions == "learned":
        w["model.embed_positions.weight"] = mat(cfg.max_positions, dm)
    gated = cfg.mlp in ("swiglu", "geglu", "geglu_tanh")
    for i in range(cfg.n_layers):
        p = "model.layers.%d." % i
        w[p + "input_layernorm.weight"] = (1 + mat(dm)).astype(np.float32)
        w[p + "post_attention_layernorm.weight"] = (1 + mat(dm)).astype(np.float32)
        w[p + "self_attn.q_proj.weight"] = mat(nh * hd, dm)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * hd, dm)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * hd, dm)
        w[p + "self_attn.o_proj.weight"] = mat(dm, nh * hd)
        w[p + "mlp.up_proj.weight"] = mat(it, dm)
        w[p + "mlp.down_proj.weight"] = mat(dm, it)
        if gated:
            w[p + "mlp.gate_proj.weight"] = mat(it, dm)
        if cfg.norm_bias:
            w[p + "input_layernorm.bias"] = mat(dm)
            w[p + "post_attention_layernorm.bias"] = mat(dm)
        if cfg.qkv_bias:
            for n_, width in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd)):
                w[p + "self_attn.%s_proj.bias" % n_] = mat(width)
        if cfg.o_bias:
            w[p + "self_attn.o_proj.bias"] = mat(dm)
        if getattr(cfg, "qk_norm", False):
            w[p + "self_attn.q_norm.weight"] = (1 + mat(hd)).astype(np.float32)
            w[p + "self_attn.k_norm.weight"] = (1 + mat(hd)).astype(np.float32)
        if cfg.mlp_bias:
            w[p + "mlp.up_proj.bias"] = mat(it)
            w[p + "mlp.down_proj.bias"] = mat(dm)
            if gated:
                w[p + "mlp.gate_proj.bias"] = mat(it)
    return w


# the block lanes of the verify table that share the `transformer` weights: (lane, weight format); the window lane
# is the same block with window = 8 (tools/identity_break.py:3639-3653, :3729-3737, :5081-5096)
LANE_FORMATS = [("transformer", "float32"), ("transformer-bf16w", "bfloat16"), ("transformer-int8w", "int8"),
                ("transformer-window", "float32")]


def lane_window(lane):
    return 8 if lane == "transformer-window" else 0


def embedding_lane(Xh):
    """The forward half of the verify table's `embedding` lane (tools/identity_break.py:7601-7621, :9530-9534): a hashed
    (128, 16) table, the 512 held-out ids of the `infer` column and the 64 of the `batch` column."""
    w = hashed_weight((128, 16), "emb:w", -0.25, 0.25)
    ids = (fixture_ids(Xh, 1, 512, 256).reshape(512) % 128).astype(np.int32)
    ids64 = (fixture_ids(Xh, 1, 64, 256).reshape(64) % 128).astype(np.int32)
    return w, ids, ids64


def rows_cell_hash(label, out):
    """A `batch` column made of one row-wise call (tools/identity_break.py:8624-8644, :8726-8727)."""
    out = np.ascontiguousarray(out)
    h = hashlib.sha256()
    h.update(("rows:%s:%d" % (label, out.shape[0])).encode())
    head = ("%s%s" % (out.dtype.str, tuple(out.shape[1:]))).encode()
    for row in out:
        h.update(head)
        h.update(row.tobytes())
    return h.hexdigest()[:16]


def lcg_floats(n, seed, lo=-0.125, hi=0.125):
    """`n` float32 values in [lo, hi) from the 64-bit LCG of the reference's synthetic checkpoints
    (python/mojolearn/_causal_lm_fixtures.py:38-47): hashed, not random, the same bytes on every machine."""
    mask = (1 << 64) - 1
    x = (seed * 6364136223846793005 + 1442695040888963407) & mask
    out = np.empty(n, np.float32)
    for i in range(n):
        x = (x * 6364136223846793005 + 1442695040888963407) & mask
        out[i] = np.float32(lo + (hi - lo) * ((x >> 11) / float(1 << 53)))
    return out


class LlamaFixtureConfig(object):
    """The Llama row of the reference's loaded-model fixtures (_causal_lm_fixtures.py:68-79): two layers, two heads
    over one KV head, head_dim 16, an untied head, a vocabulary of 64."""
    vocab, d_model, n_layers, n_heads, n_kv_heads, head_dim, intermediate = 64, 32, 2, 2, 1, 16, 64
    norm, norm_eps, norm_bias, mlp, mlp_bias, qkv_bias, o_bias = "rmsnorm", 1e-6, False, "swiglu", False, False, False
    positions, rope_theta, max_positions, window = "rope", 10000.0, 128, 0


def llama_fixture_weights(seed=1):
    """The tensors of that checkpoint (_causal_lm_fixtures.py:81-102), by HuggingFace name."""
    c = LlamaFixtureConfig
    dm, nh, nkv, hd, it, v = c.d_model, c.n_heads, c.n_kv_heads, c.head_dim, c.intermediate, c.vocab

    def f32(shape, sd, lo=-0.125, hi=0.125):
        return lcg_floats(shape[0] * shape[1], sd, lo, hi).reshape(shape)

    w = {"model.embed_tokens.weight": f32((v, dm), seed + 1, -0.5, 0.5), "model.norm.weight": np.ones(dm, np.float32),
         "lm_head.weight": f32((v, dm), seed + 2, -0.5, 0.5)}
    for i in range(c.n_layers):
        p, s = "model.layers.%d." % i, seed + 10 * (i + 1)
        w[p + "input_layernorm.weight"] = np.ones(dm, np.float32)
        w[p + "post_attention_layernorm.weight"] = np.ones(dm, np.float32)
        w[p + "self_attn.q_proj.weight"] = f32((nh * hd, dm), s + 1)
        w[p + "self_attn.k_proj.weight"] = f32((nkv * hd, dm), s + 2)
        w[p + "self_attn.v_proj.weight"] = f32((nkv * hd, dm), s + 3)
        w[p + "self_attn.o_proj.weight"] = f32((dm, nh * hd), s + 4)
        w[p + "mlp.gate_proj.weight"] = f32((it, dm), s + 5)
        w[p + "mlp.up_proj.weight"] = f32((it, dm), s + 6)
        w[p + "mlp.down_proj.weight"] = f32((dm, it), s + 7)
    return w


def fixture_ids(X, b, l, vocab):
    """A (b, l) int32 token stream: the first b*l BYTES of the fixture, modulo the vocabulary
    (the verify table's hf-causal-lm lane, tools/identity_break.py:3038-3044)."""
    raw = np.frombuffer(np.ascontiguousarray(X).tobytes()[: b * l], dtype=np.uint8)
    return np.ascontiguousarray((raw.astype(np.int32) % vocab).reshape(b, l))


def batch_cell_hash_block(y):
    """The verify table's `batch` column of a block forward over a (B, L, d) slab (tools/identity_break.py:9591-9604):
    the whole-batch rows, then the whole output as the full-length answer of the prefix part."""
    y = np.ascontiguousarray(y)
    b, l, d = y.shape
    h = hashlib.sha256()
    h.update(("rows:forward:%d" % b).encode())
    for i in range(b):
        h.update(("<f4(%d, %d)" % (l, d)).encode())
        h.update(y[i].tobytes())
    h.update(("prefix:forward:%d:1" % l).encode())
    h.update(("<f4(%d, %d, %d)" % (b, l, d)).encode())
    h.update(y.tobytes())
    return h.hexdigest()[:16]


def decode_session_parts(steps, prefill, k_cache, v_cache):
    """The parts of the `transformer-decode-session` lane (tools/identity_break.py:8239-8272): the 16 stepped outputs,
    the chunked prefill, the resident caches as the reference's flat host buffers, and the six refusal flags (all
    true). `oracle.train_hash` of the result is the lane's `train` cell."""
    import lanes
    flags = np.ones(6, dtype=np.int64)
    return dict(step=lanes.sha16(*steps), prefill=lanes.sha16(prefill), state=lanes.sha16(k_cache, v_cache), flags=lanes.sha16(flags))


def packed_cache(cache, used):
    """[B, KV, cap, HD] -> the reference's flat state buffer: the used positions packed as [B, KV, used, HD], then
    spare zeros (python/mojolearn/_transformer_impl.py:194-213)."""
    cache = np.asarray(cache, dtype=np.float32)
    flat = np.zeros(cache.size, dtype=np.float32)
    part = np.ascontiguousarray(cache[:, :, :used, :]).reshape(-1)
    flat[:part.size] = part
    return flat


def stepfull_cell_hash(y, how="allocate_state + step"):
    """The verify table's `stepfull` column of a block (tools/identity_break.py:10345-10382, :10402-10430): one
    fresh-state forward over (2, 16, d) hashed under the call's label; valid when one step per position (per-call,
    or through a decode session) reproduces it."""
    y = np.ascontiguousarray(y)
    h = hashlib.sha256()
    h.update(("stepfull:forward(x) vs %s, L=%d:%s" % (how, y.shape[1], list(y.shape))).encode())
    h.update(("<f4%s" % (tuple(y.shape),)).encode())
    h.update(y.tobytes())
    return h.hexdigest()[:16]


RAGGED_LENGTHS = (16, 1, 7, 9, 16, 3, 12, 15)
RAGGED_LONG_LENGTHS = (300, 1, 65, 129, 257, 128)


def tiled(X, shape):
    """`shape` float32 values from the fixture, row-major and wrapped (tools/identity_break.py:10054-10058)."""
    return np.ascontiguousarray(np.resize(np.ascontiguousarray(X).reshape(-1), int(np.prod(shape))).reshape(shape))


def ragged_inputs(Xh, dm):
    """The two ragged calls of a block (tools/identity_break.py:10249-10257): junk (NaN) at the padding positions."""
    calls = []
    for x, lens in ((seq(Xh, len(RAGGED_LENGTHS), 16, dm), RAGGED_LENGTHS),
                    (tiled(Xh, (len(RAGGED_LONG_LENGTHS), max(RAGGED_LONG_LENGTHS), dm)), RAGGED_LONG_LENGTHS)):
        x = np.array(x, dtype=np.float32, copy=True)
        for i, n in enumerate(lens):
            x[i, n:] = np.float32("nan")
        calls.append((x, lens))
    return calls


def ragged_cell_hash(outs):
    """The verify table's `ragged` column (tools/identity_break.py:10207-10234): per call a label with the input shape
    and the lengths, then the padded output; valid when every row's real positions equal the row alone and the
    padding is exactly +0.0, which the tests hold separately. `outs` = [(x, lengths, y), ...]."""
    h = hashlib.sha256()
    for x, lens, y in outs:
        y = np.ascontiguousarray(y)
        h.update(("ragged:forward(lengths) L=%d:%s:%s" % (x.shape[1], list(x.shape), tuple(lens))).encode())
        h.update(("<f4%s" % (tuple(y.shape),)).encode())
        h.update(y.tobytes())
    return h.hexdigest()[:16]


def batchscale_inputs(Xh, dm):
    """The serving-size calls of a block (tools/identity_break.py:10086-10093) at the sizes the committed table was
    recorded with (1024 rows and a long length of 1024; the harness has since shrunk both, :9989-9995, :10084):
    1024 rows of 16 positions, and two rows of 1024 positions cut from the reversed fixture."""
    return tiled(Xh, (1024, 16, dm)), tiled(Xh[::-1], (2, 1024, dm))


def batchscale_cell_hash(y_rows, y_long):
    """The verify table's `batchscale` column of a block (tools/identity_break.py:10018-10052, :8731-8767): the
    1024-row call's rows under the sub-batch sizes it was asked at (1, 17, 64, 256), then the 1024-position call as
    the full-length answer of its prefix part."""
    y_rows, y_long = np.ascontiguousarray(y_rows), np.ascontiguousarray(y_long)
    n, l, d = y_rows.shape
    h = hashlib.sha256()
    h.update(("scale:forward L=%d:%d:1,17,64,256" % (l, n)).encode())
    for i in range(n):
        h.update(("<f4(%d, %d)" % (l, d)).encode())
        h.update(y_rows[i].tobytes())
    h.update(("prefix:forward B=2 L=%d:%d:1" % (y_long.shape[1], y_long.shape[1])).encode())
    h.update(("<f4%s" % (tuple(y_long.shape),)).encode())
    h.update(y_long.tobytes())
    return h.hexdigest()[:16]


SCALE_PREFIXES = (1, 7, 63, 64, 65, 127, 128, 129, 255, 256, 257, 511, 513, 1023)


def batch_cell_hash(logits):
    """The verify table's `batch` column for a causal LM forward over (B, L) ids (tools/identity_break.py:8624-8644,
    :8731-8767, :9446-9460): sha256 over the whole-batch rows (each with its dtype and shape) and then the whole
    output as the full-length answer of the prefix part; valid when every row alone, every split and every prefix
    reproduces the whole batch's bytes, which the tests hold separately."""
    logits = np.ascontiguousarray(logits)
    b, l, v = logits.shape
    h = hashlib.sha256()
    h.update(("rows:forward:%d" % b).encode())
    for i in range(b):
        h.update(("<f4(%d, %d)" % (l, v)).encode())
        h.update(logits[i].tobytes())
    h.update(("prefix:forward:%d:1" % l).encode())
    h.update(("<f4(%d, %d, %d)" % (b, l, v)).encode())
    h.update(logits.tobytes())
    return h.hexdigest()[:16]


class OracleLM(object):
    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights
        self.bcfg = oracle.block_cfg(cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.intermediate, norm=cfg.norm,
                                     norm_eps=cfg.norm_eps, norm_bias=cfg.norm_bias, qkv_bias=cfg.qkv_bias, o_bias=cfg.o_bias,
                                     mlp=cfg.mlp, mlp_bias=cfg.mlp_bias, rope=cfg.positions == "rope",
                                     rope_theta=cfg.rope_theta, window=cfg.window, rope_scaling=getattr(cfg, "rope_scaling", None),
                                     rope_dim=getattr(cfg, "rope_dim", None), qk_norm=getattr(cfg, "qk_norm", False),
                                     attn_softcap=getattr(cfg, "attn_softcap", None))
        self.slots = [block_slots(weights, "model.layers.%d." % i) for i in range(cfg.n_layers)]

    def allocate_state(self, b, cap):
        return [oracle.KVState(b, self.cfg.n_kv_heads, cap, self.cfg.head_dim) for _ in range(self.cfg.n_layers)]

    def forward(self, ids, state=None):
        ids = np.asarray(ids, dtype=np.int32)
        b, l = ids.shape
        if state is None:
            state = self.allocate_state(b, l)
        x = oracle.embedding(self.w["model.embed_tokens.weight"], ids)
        if self.cfg.positions == "learned":
            x = oracle.add_positions(x, self.w["model.embed_positions.weight"], state[0].used)
        for slots, st in zip(self.slots, state):
            x = oracle.block_forward(self.bcfg, slots, x, st)
        hn = oracle.norm(x.reshape(b * l, -1), self.w["model.norm.weight"], self.w.get("model.norm.bias"), self.cfg.norm_eps,
                         self.cfg.norm)
        return oracle.gemm_rows(hn, self.w["lm_head.weight"], oracle.OP_NT).reshape(b, l, -1)

    def generate(self, ids, new_tokens):
        ids = np.asarray(ids, dtype=np.int32)
        b, l = ids.shape
        state = self.allocate_state(b, l + new_tokens)
        logits = self.forward(ids, state)[:, -1, :]
        out, kept = [ids], []
        for step in range(new_tokens):
            nxt = oracle.argmax(logits).reshape(b, 1)
            out.append(nxt)
            kept.append(logits)
            if step + 1 < new_tokens:
                logits = self.forward(nxt, state)[:, -1, :]
        return np.concatenate(out, axis=1), np.stack(kept, axis=1)

"""The two decoder benchmark configurations at their stated size, one sequence held to the CPU oracle.

Configuration 4: 12 layers, d_model 768, 12 heads, MLP 3072 GELU, LayerNorm, learned positions, vocabulary 50304,
float32 weights N(0, 0.02), batch 8, a 512-token prompt then 128 greedy steps. Configuration 5 (the serving
benchmark): 24 layers, d_model 2048, 16 heads of 128, MLP 8192, INT8 weights with per-row power-of-two exponents,
batch 32, a 1024-token prompt then 256 greedy steps, built with the benchmark's own weight and id generators.

The CUDA path runs the whole batch through `CausalLM.generate` (prefill, then the decode step replayed from its CUDA
graph: the kernels the benchmark times). The oracle then reads sequence 0 of the generated ids as ONE teacher-forced
forward over prompt + continuation. Its logits at position 1023 + t are what the oracle's own t-th decode step would
produce (a position's row reads only earlier keys, and every product cell is independent of the rows beside it:
tests/test_oracle_decoder.py holds the oracle's step to its forward), so comparing them with the logits the CUDA path
produced at step t, and their argmax with the generated ids, is the greedy continuation compared step by step
(transformer/IDENTICAL_TRANSFORMER_CONTRACT.md:540-565 of the reference: decode equals prefill). Bit for bit.
"""
import numpy as np
import pytest

import decoder_ref
import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import serve_bench  # noqa: E402
from mojolearn_b200.models import CausalLM, CausalLMConfig  # noqa: E402


oracle_teacher_forced = oracle.teacher_forced_logits


def check_continuation(seq_row, kept_row, want_logits, prompt):
    """seq_row [prompt + steps], kept_row [steps, vocab] from the CUDA path; want_logits [steps, vocab] from the oracle."""
    steps = kept_row.shape[0]
    for t in range(steps):
        assert kept_row[t].tobytes() == want_logits[t].tobytes(), "logits of decode step %d differ from the oracle" % t
    assert oracle.argmax(want_logits).tolist() == [int(v) for v in seq_row[prompt:prompt + steps]]


def test_config4_full_size_sequence_against_the_oracle():
    cfg = CausalLMConfig(vocab=50304, d_model=768, n_layers=12, n_heads=12, intermediate=3072, norm="layernorm", norm_bias=True,
                         mlp="gelu", mlp_bias=True, qkv_bias=True, o_bias=True, positions="learned", max_positions=640)
    w = decoder_ref.random_lm_weights(cfg, seed=0, scale=0.02)
    prompt, steps, batch = 512, 128, 8
    ids = np.random.default_rng(0).integers(0, cfg.vocab, (batch, prompt)).astype(np.int32)
    seq, kept = CausalLM(cfg, w).generate(ids, steps, return_logits=True)
    assert seq.shape == (batch, prompt + steps) and kept.shape == (batch, steps, cfg.vocab)
    for row in (0, batch - 1):
        want = oracle_teacher_forced(cfg, seq[row, :prompt + steps - 1], prompt - 1,
                                     lambda i: decoder_ref.block_slots(w, "model.layers.%d." % i), w["model.embed_tokens.weight"],
                                     w["model.embed_positions.weight"], w["model.norm.weight"], w["model.norm.bias"],
                                     w["lm_head.weight"])
        check_continuation(seq[row], kept[row], want, prompt)


def test_config5_full_size_sequence_against_the_oracle():
    cfg = CausalLMConfig(vocab=50304, d_model=2048, n_layers=24, n_heads=16, intermediate=8192, max_positions=8192)
    w = serve_bench.build_weights(cfg, "int8")  # the benchmark's weights: device-resident int8 codes and row exponents
    prompt, steps, batch = 1024, 256, 32
    ids = serve_bench.build_ids(cfg, batch, prompt)  # and its token ids
    lm = CausalLM(cfg, w)
    seq, kept = lm.generate(ids, steps, return_logits=True)
    seq0, kept0 = seq[0].cpu().numpy(), kept[0].cpu().numpy()
    del kept, lm
    torch.cuda.empty_cache()

    def host(layer):  # int8 codes and exponents of a device Linear -> the exact float32 weight the product reads
        return oracle.dequantize_int8(layer.w.cpu().numpy(), layer.scale.cpu().numpy())

    def slots(i):
        p = "model.layers.%d." % i
        names = dict(q="self_attn.q_proj", k="self_attn.k_proj", v="self_attn.v_proj", o="self_attn.o_proj",
                     gate="mlp.gate_proj", up="mlp.up_proj", down="mlp.down_proj")
        out = {slot: host(w[p + name + ".weight"]) for slot, name in names.items()}
        out["norm1"] = w[p + "input_layernorm.weight"].cpu().numpy()
        out["norm2"] = w[p + "post_attention_layernorm.weight"].cpu().numpy()
        return out

    want = oracle_teacher_forced(cfg, seq0[:prompt + steps - 1], prompt - 1, slots, w["model.embed_tokens.weight"].cpu().numpy(),
                                 None, w["model.norm.weight"].cpu().numpy(), None, host(w["lm_head.weight"]))
    check_continuation(seq0, kept0, want, prompt)

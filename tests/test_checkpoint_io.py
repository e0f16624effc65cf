"""Checkpoint reading on the host: the safetensors container, exact widening of F16 / BF16, sharded indexes, and the
config -> plan mapping with its refusals by name (reference python/mojolearn/models/safetensors.py, models/config.py)."""
import json
import os
import struct

import numpy as np
import pytest

from mojolearn_b200 import lowbit
from mojolearn_b200.models import config, safetensors


def test_f16_widening_is_exact_on_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    got = safetensors.widen_f16(bits)
    want = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    assert np.isnan(got[nan]).all() and np.array_equal(np.signbit(got[nan]), np.signbit(want[nan]))


def test_roundtrip_single_file_and_storage_types(tmp_path):
    rng = np.random.default_rng(0)
    f32 = rng.standard_normal((5, 7)).astype(np.float32)
    i32 = rng.integers(-9, 9, (4,)).astype(np.int32)
    i64 = rng.integers(-9, 9, (2, 3)).astype(np.int64)
    bf = (rng.standard_normal((6, 8)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    path = tmp_path / "model.safetensors"
    safetensors.write_file(path, {"a": f32, "b": i32, "c": i64, "w": bf})
    with safetensors.SafetensorsFile(path) as f:
        assert f.names() == ["a", "b", "c", "w"] and f.info("w").dtype == "BF16" and f.info("a").shape == (5, 7)
        assert f.read("a").tobytes() == f32.tobytes() and f.read("b").tobytes() == i32.tobytes() and f.read("c").tobytes() == i64.tobytes()
        wide = f.read("w")
        assert wide.dtype == np.float32 and wide.view(np.uint32).tobytes() == (bf.astype(np.uint32) << 16).tobytes()
        kept = f.read("w", bf16="bits")
        assert isinstance(kept, lowbit.BF16Weight) and kept.bits.tobytes() == bf.tobytes()
        with pytest.raises(KeyError):
            f.read("missing")
    # an F16 tensor and an unread storage type, written by hand
    half = rng.standard_normal((3, 2)).astype(np.float16)
    header = {"h": {"dtype": "F16", "shape": [3, 2], "data_offsets": [0, 12]}, "u": {"dtype": "U8", "shape": [4], "data_offsets": [12, 16]}}
    text = json.dumps(header).encode()
    p2 = tmp_path / "other.safetensors"
    with open(p2, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)) + text + half.tobytes() + bytes(4))
    f2 = safetensors.SafetensorsFile(p2)
    assert f2.read("h").tobytes() == half.astype(np.float32).tobytes()
    with pytest.raises(TypeError, match="U8"):
        f2.read("u")
    with open(tmp_path / "short.safetensors", "wb") as fh:
        fh.write(b"abc")
    with pytest.raises(ValueError):
        safetensors.SafetensorsFile(tmp_path / "short.safetensors")


def test_sharded_checkpoint(tmp_path):
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.arange(4, dtype=np.float32)
    safetensors.write_file(tmp_path / "s1.safetensors", {"a": a})
    safetensors.write_file(tmp_path / "s2.safetensors", {"b": b})
    json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}, open(tmp_path / safetensors.INDEX_NAME, "w"))
    with safetensors.Checkpoint.open(tmp_path) as ck:
        assert ck.names() == ["a", "b"] and "a" in ck and "z" not in ck
        assert ck.read("a").tobytes() == a.tobytes() and ck.read("b").tobytes() == b.tobytes() and ck.info("b").shape == (4,)
    with pytest.raises(FileNotFoundError):
        safetensors.Checkpoint.open(tmp_path / "nowhere")


BASE = {"model_type": "llama", "vocab_size": 64, "hidden_size": 32, "num_hidden_layers": 2, "num_attention_heads": 2,
        "num_key_value_heads": 1, "intermediate_size": 64, "rms_norm_eps": 1e-5, "rope_theta": 500000.0}


def test_plan_for_families_and_refusals():
    plan = config.plan_for(BASE)
    assert (plan.vocab, plan.d_model, plan.n_layers, plan.n_heads, plan.n_kv_heads, plan.head_dim) == (64, 32, 2, 2, 1, 16)
    assert plan.norm_eps == 1e-5 and plan.rope_theta == 500000.0 and not plan.qkv_bias and not plan.qk_norm
    assert config.plan_for(dict(BASE, model_type="qwen2")).qkv_bias and config.plan_for(dict(BASE, model_type="qwen3")).qk_norm
    assert config.plan_for(dict(BASE, model_type="mistral", sliding_window=8)).window == 8
    scaled = config.plan_for(dict(BASE, rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}))
    assert scaled.rope_scaling["rope_type"] == "llama3"
    assert config.plan_for(dict(BASE, partial_rotary_factor=0.5)).rope_dim == 8
    for bad, word in ((dict(BASE, model_type="mamba"), "mamba"), (dict(BASE, hidden_act="gelu"), "hidden_act"),
                      (dict(BASE, rope_scaling={"rope_type": "yarn", "factor": 2.0}), "yarn"),
                      ({k: v for k, v in BASE.items() if k != "vocab_size"}, "vocab_size")):
        with pytest.raises(config.UnsupportedModel, match=word):
            config.plan_for(bad)
    names = config.checkpoint_names(config.plan_for(dict(BASE, model_type="qwen3", tie_word_embeddings=True)))
    assert "lm_head.weight" not in names and "model.layers.1.self_attn.k_norm.weight" in names

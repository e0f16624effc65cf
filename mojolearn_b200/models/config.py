"""A Hugging Face `config.json` to a `CausalLMConfig`, family by family.

Mirrors python/mojolearn/models/config.py of the reference (the option matrix, :45-75, and the family rows,
:208-219) for the transformer families the block spells: llama (Llama 2/3, TinyLlama, SmolLM), mistral
(sliding_window -> window), qwen2 (qkv_bias), qwen3 (qk_norm). Every field the blocks cannot honor is refused BY
NAME with its value, never run at a different setting. The Mamba rows, phi3's fused projections and the gemma rows of
the reference are outside this package's path and are refused by model_type.
"""
import json
import os

from .causal_lm import CausalLMConfig

POSITION_CEILING = 8192
FAMILIES = ("llama", "smollm", "mistral", "qwen2", "qwen3")


class UnsupportedModel(ValueError):
    """A config field the blocks cannot honor, refused by name."""


def read_config(path):
    """`path` is `config.json` or the directory holding it."""
    path = str(path)
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as f:
        return json.load(f)


def plan_for(cfg):
    """The `CausalLMConfig` of a config dict, or an `UnsupportedModel` naming the model type or field."""
    mt = cfg.get("model_type")
    if mt not in FAMILIES:
        raise UnsupportedModel("model_type %r is not a family this package loads (%s are)" % (mt, ", ".join(FAMILIES)))

    def need(key):
        if key not in cfg:
            raise UnsupportedModel("%s config lacks %r" % (mt, key))
        return cfg[key]

    act = cfg.get("hidden_act", "silu")
    if act != "silu":
        raise UnsupportedModel("%s: hidden_act %r is not spelled (silu, the gated SwiGLU, is)" % (mt, act))
    if cfg.get("attention_bias", False) and mt not in ("qwen2",):
        qkv_bias = o_bias = True
    else:
        qkv_bias, o_bias = mt == "qwen2", False
    if cfg.get("mlp_bias", False):
        mlp_bias = True
    else:
        mlp_bias = False
    scaling = cfg.get("rope_scaling")
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind not in (None, "default", "linear", "llama3"):
            raise UnsupportedModel("%s: rope_scaling %r is not spelled (linear and llama3 are)" % (mt, kind))
        if kind in (None, "default"):
            scaling = None
    window = 0
    if mt == "mistral" and cfg.get("sliding_window"):
        window = int(cfg["sliding_window"])
    if mt in ("qwen2", "qwen3") and cfg.get("use_sliding_window", False):
        raise UnsupportedModel("%s: use_sliding_window with max_window_layers is not spelled" % mt)
    n_heads = int(need("num_attention_heads"))
    d_model = int(need("hidden_size"))
    head_dim = int(cfg.get("head_dim") or d_model // n_heads)
    partial = float(cfg.get("partial_rotary_factor", 1.0))
    rope_dim = int(head_dim * partial)
    max_pos = min(int(cfg.get("max_position_embeddings", POSITION_CEILING)), POSITION_CEILING *
                  (int(scaling["factor"]) if scaling and scaling.get("rope_type", scaling.get("type")) == "linear" else 1))
    return CausalLMConfig(vocab=int(need("vocab_size")), d_model=d_model, n_layers=int(need("num_hidden_layers")), n_heads=n_heads,
                          n_kv_heads=int(cfg.get("num_key_value_heads") or n_heads), head_dim=head_dim,
                          intermediate=int(need("intermediate_size")), norm="rmsnorm", norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
                          mlp="swiglu", mlp_bias=mlp_bias, qkv_bias=qkv_bias, o_bias=o_bias, positions="rope",
                          rope_theta=float(cfg.get("rope_theta", 10000.0)), max_positions=max_pos, window=window,
                          rope_scaling=scaling, rope_dim=rope_dim if rope_dim != head_dim else None, qk_norm=mt == "qwen3",
                          tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)))


def checkpoint_names(plan):
    """Every tensor name a checkpoint of this plan must hold."""
    names = ["model.embed_tokens.weight", "model.norm.weight"]
    if not plan.tie_word_embeddings:
        names.append("lm_head.weight")
    for i in range(plan.n_layers):
        p = "model.layers.%d." % i
        names += [p + "input_layernorm.weight", p + "post_attention_layernorm.weight"]
        names += [p + "self_attn.%s_proj.weight" % s for s in "qkvo"] + [p + "mlp.%s_proj.weight" % s for s in ("gate", "up", "down")]
        if plan.qkv_bias:
            names += [p + "self_attn.%s_proj.bias" % s for s in "qkv"]
        if plan.o_bias:
            names.append(p + "self_attn.o_proj.bias")
        if plan.mlp_bias:
            names += [p + "mlp.%s_proj.bias" % s for s in ("gate", "up", "down")]
        if plan.qk_norm:
            names += [p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight"]
    return names

"""`TransformerBlock`: the reference's decoder block on B200, device resident.

Mirrors python/mojolearn/_transformer_impl.py of the reference (:408-419 the
constructor and its options, :461-481 `forward`, :527-572 `step` and
`allocate_state`, :195-216 the state): weights by HuggingFace names in torch
`[out, in]` layout, either float32 arrays or `lowbit`-packed (bf16 bits, or int8
codes with per-row power-of-two exponents), which are materialised exactly inside
the product kernels. Every projection is a `gemm.fp32.v1` OP_NT product; every
other step is the reference's pinned seam (see csrc/decoder.cuh). A decode step
is the same entry at L = 1 and equals the prefill bit for bit.

`rope=False` and learned positions are an extension: the reference's block
always rotates (transformer/block_options.mojo:46-48).

Activations may be numpy arrays (copied to the device and back, like the
reference's host surface) or CUDA torch tensors (stay on the device).
"""
import ctypes
import os

import numpy as np
import torch

from . import _native, _prof, lowbit
from .linalg import OP_NT, W_BF16, W_F32, W_INT8_EXP, W_INT8_SCALE
from . import torch_ops
from .parallel import gather_columns, shard_bounds

NORM_KINDS = {"rmsnorm": 0, "layernorm": 1, "rmsnorm_offset": 2}
MLP_KINDS = {"swiglu": 0, "silu_gated": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "geglu": 4, "geglu_tanh": 5}
GATED = (0, 4, 5)
MAX_POSITIONS = 8192


def _vp(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _vector(x, name, device):
    """A float32 tensor on the device from a numpy array or a torch tensor; non-finite values are refused by name."""
    if isinstance(x, torch.Tensor):
        t = x.to(device=device, dtype=torch.float32).contiguous()
        if not bool(torch.isfinite(t).all()):
            raise ValueError("non-finite values in %s REFUSED" % name)
        return t
    a = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    if not np.isfinite(a).all():
        raise ValueError("non-finite values in %s REFUSED" % name)
    return torch.from_numpy(a).to(device)


class Linear(object):
    """One `[out, in]` weight on the device in its storage format, applied as x @ W^T."""

    def __init__(self, w, device, bias=None, rows=None):
        if isinstance(w, Linear):
            self.__dict__.update(w.__dict__)
            return
        self.scale = None
        if isinstance(w, lowbit.BF16Weight):
            self.w, self.kind = torch.from_numpy(np.ascontiguousarray(w.bits)).to(device), W_BF16
        elif isinstance(w, lowbit.Int8Weight):
            self.w, self.kind = torch.from_numpy(np.ascontiguousarray(w.codes)).to(device), W_INT8_EXP
            self.scale = torch.from_numpy(np.ascontiguousarray(w.exponents)).to(device)
        elif isinstance(w, tuple) and len(w) == 2:  # (int8 codes, float32 scales): the extension format
            self.w, self.kind = torch.as_tensor(np.ascontiguousarray(w[0])).to(device), W_INT8_SCALE
            self.scale = torch.as_tensor(np.ascontiguousarray(w[1], dtype=np.float32)).to(device)
        else:
            a = w if isinstance(w, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(np.asarray(w)))
            if a.dtype != torch.float32 or a.dim() != 2:
                raise TypeError("a projection weight must be 2-D float32 (or a lowbit-packed weight)")
            self.w, self.kind = a.to(device).contiguous(), W_F32
        self.bias = None
        if bias is not None:
            self.bias = torch.as_tensor(np.ascontiguousarray(np.asarray(bias, dtype=np.float32))).to(device)
        self.out_features, self.in_features = self.w.shape

    @classmethod
    def from_device(cls, w, scale=None, kind=W_F32, bias=None):
        """A layer over tensors that already live on the device (weights built or quantised there)."""
        self = cls.__new__(cls)
        self.w, self.scale, self.kind, self.bias = w.contiguous(), scale, kind, bias
        self.out_features, self.in_features = self.w.shape
        return self

    @classmethod
    def concat(cls, parts):
        """One layer whose output columns are those of `parts` side by side (weight rows stacked), or None when
        the parts differ in storage kind, width or in having a bias. Bit-neutral: a product cell reads one
        weight row, so which launch computes it does not matter."""
        first = parts[0]
        if any(type(p) is not Linear or p.kind != first.kind or p.in_features != first.in_features or
               (p.bias is None) != (first.bias is None) for p in parts):
            return None
        self = cls.__new__(cls)
        self.w, self.kind = torch.cat([p.w for p in parts], dim=0).contiguous(), first.kind
        self.scale = torch.cat([p.scale for p in parts]).contiguous() if first.scale is not None else None
        self.bias = torch.cat([p.bias for p in parts]).contiguous() if first.bias is not None else None
        self.out_features, self.in_features = self.w.shape
        return self

    @classmethod
    def interleave(cls, first, second):
        """One layer whose output columns alternate between the two parts' (weight row 2j = first's row j, row 2j + 1 =
        second's), or None when the parts differ in storage kind, shape or in having a bias. Bit-neutral like
        `concat`; the layout puts a gated MLP's gate_j and up_j in adjacent product columns, where one thread of the
        skinny plans owns both and can apply the gated activation as it stores."""
        if (type(first) is not Linear or type(second) is not Linear or first.kind != second.kind or first.w.shape != second.w.shape or
                (first.bias is None) != (second.bias is None)):
            return None
        self = cls.__new__(cls)
        n, k = first.w.shape
        self.w, self.kind = torch.stack([first.w, second.w], dim=1).reshape(2 * n, k).contiguous(), first.kind
        self.scale = torch.stack([first.scale, second.scale], dim=1).reshape(2 * n).contiguous() if first.scale is not None else None
        self.bias = torch.stack([first.bias, second.bias], dim=1).reshape(2 * n).contiguous() if first.bias is not None else None
        self.out_features, self.in_features = self.w.shape
        return self

    def shard_rows(self, lo, hi):
        """The same layer restricted to output rows [lo, hi): a bit-neutral shard (a cell reads one weight row)."""
        part = Linear.__new__(Linear)
        part.__dict__.update(self.__dict__)
        part.w = self.w[lo:hi].contiguous()
        part.scale = self.scale[lo:hi].contiguous() if self.scale is not None else None
        part.bias = self.bias[lo:hi].contiguous() if self.bias is not None else None
        part.out_features = hi - lo
        return part

    def __call__(self, x2d, act=0):
        """x @ W^T (+ bias) (then the ungated activation `act` of torch_ops.ACT_*), the bias and the activation
        applied where the product stores its output."""
        with _prof.span("product"):
            return torch_ops.product(x2d, self.w, self.scale, self.kind, OP_NT, bias=self.bias, act=act)


_FOLD_IN_GATHER = os.environ.get("MOJOLEARN_B200_FOLD_IN_GATHER", "1") != "0"  # 0: fold launch and gather launch apart (for timing the difference)


def product_gather(lin, x2d, act, group, exchange):
    """A rank's column slice `lin` of a sharded layer applied to x2d, gathered over the ranks. When the exchange takes
    the slice, a product that the plan split into leaf groups is left as nodes and the gather kernel folds, finishes and
    sends them itself (one launch fewer per sharded product of a decode step; the same words either way). `act` may be a
    gated pair code (the slice then has half the layer's columns)."""
    m = x2d.shape[0]
    w = lin.out_features // 2 if act >= torch_ops.ACT_PAIR_SWIGLU else lin.out_features
    if (_FOLD_IN_GATHER and exchange is not None and hasattr(exchange, "gather_nodes") and lin.out_features % 4 == 0 and x2d.dtype == torch.float32 and
            x2d.is_contiguous() and exchange.takes_shape(m, w)):
        with _prof.span("product"):
            part, ws, nodes = torch_ops.product_nodes(x2d, lin.w, lin.scale, lin.kind, bias=lin.bias, act=act)
        with _prof.span("gather"):
            if nodes > 1:
                return exchange.gather_nodes(ws, nodes, m, lin.out_features, lin.bias, act)
            return exchange.gather(part)
    with _prof.span("product"):
        part = torch_ops.product(x2d, lin.w, lin.scale, lin.kind, OP_NT, bias=lin.bias, act=act)
    with _prof.span("gather"):
        return gather_columns(part, group, exchange)  # pure data movement: no arithmetic order is introduced


class ShardedLinear(object):
    """Rows [r*N/g, (r+1)*N/g) of a layer on this rank; the call all-gathers the output columns."""

    def __init__(self, full, group, rank, world, exchange=None):
        n = full.out_features
        lo, hi = shard_bounds(n, rank, world)
        self.local = full.shard_rows(lo, hi)
        self.group, self.world, self.out_features, self.in_features = group, world, n, full.in_features
        self.exchange = exchange

    def __call__(self, x2d, act=0):
        return product_gather(self.local, x2d, act, self.group, self.exchange)


class TransformerState(object):
    """Caller-owned KV caches `[B, n_kv_heads, max_tokens, head_dim]` float32 on the device and the tokens cached
    (the reference's state, `_transformer_impl.py:194-236`; its host buffers are packed at stride `cached_tokens`,
    which `k_cache` / `v_cache` below reproduce on request). `window` records the sliding window the state was
    allocated for; a session checks it against the block's."""

    def __init__(self, batch, n_kv_heads, max_tokens, head_dim, device, window=0):
        self.k = torch.zeros((batch, n_kv_heads, max_tokens, head_dim), dtype=torch.float32, device=device)
        self.v = torch.zeros_like(self.k)
        self.cached_tokens = 0
        self.max_tokens = max_tokens
        self.window = int(window or 0)
        self.session = None  # the open decode session that owns this state, if any

    @property
    def batch_size(self):
        return self.k.shape[0]

    def clone(self):
        other = TransformerState.__new__(TransformerState)
        other.k, other.v = self.k.clone(), self.v.clone()
        other.cached_tokens, other.max_tokens, other.window, other.session = self.cached_tokens, self.max_tokens, self.window, None
        return other

    def keys(self):
        """The used part of the key cache, (B, n_kv_heads, cached_tokens, head_dim), as a host array."""
        return self.k[:, :, :self.cached_tokens, :].contiguous().cpu().numpy()

    def values(self):
        return self.v[:, :, :self.cached_tokens, :].contiguous().cpu().numpy()

    def _packed(self, cache):
        flat = np.zeros(cache.numel(), dtype=np.float32)
        used = cache[:, :, :self.cached_tokens, :].contiguous().cpu().numpy().reshape(-1)
        flat[:used.size] = used
        return flat

    @property
    def k_cache(self):
        """The reference's flat host buffer: the used keys packed as [B, KV, cached_tokens, HD], then spare zeros."""
        return self._packed(self.k)

    @property
    def v_cache(self):
        return self._packed(self.v)


class TransformerDecodeSession(object):
    """A resident decode session over one block and one state (the reference's `TransformerBlock.decode_session`,
    `_transformer_impl.py:609-633`). Every output is byte for byte the per-call `step` / `forward` on the same
    block and state: here the state already lives on the device between calls, so the session is the ownership
    protocol around it (one open session per state, a fixed batch size, the block's window) and `sync_state`
    only waits for the device."""

    def __init__(self, block, state):
        self.block, self.state, self.is_open = block, state, True
        state.session = self

    def _check(self, x):
        if not self.is_open:
            raise RuntimeError("the decode session is closed")
        if x.shape[0] != self.state.batch_size:
            raise ValueError("the session was opened for %d sequences, got %d" % (self.state.batch_size, x.shape[0]))

    def step(self, x):
        self._check(x)
        return self.block.step(x, self.state)

    def forward(self, x):
        self._check(x)
        return self.block.forward(x, self.state)

    def sync_state(self):
        torch.cuda.synchronize(self.block.device)
        return self.state

    def close(self):
        if self.is_open:
            self.is_open = False
            self.state.session = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def norm(x2d, w, bias, eps, kind):
    out = torch.empty_like(x2d)
    dev = x2d.device
    with _prof.span("norm"):
        return _norm(out, x2d, w, bias, eps, kind, dev)


def _norm(out, x2d, w, bias, eps, kind, dev):
    _native.call("b200i_norm", dev.index, _stream(dev), _vp(out), _vp(x2d), _vp(w), _vp(bias), x2d.shape[0], x2d.shape[1],
                 float(eps), kind)
    return out


def add_norm(x2d, delta, w, bias, eps, kind):
    """(x + delta, norm(x + delta)): the residual add and the norm that follows it, one pass over the rows."""
    out, total = torch.empty_like(x2d), torch.empty_like(x2d)
    dev = x2d.device
    with _prof.span("norm"):
        _native.call("b200i_add_norm", dev.index, _stream(dev), _vp(out), _vp(total), _vp(x2d), _vp(delta.contiguous()), _vp(w), _vp(bias),
                     x2d.shape[0], x2d.shape[1], float(eps), kind)
    return total, out


def add(a, b):
    out = torch.empty_like(a)
    dev = a.device
    _native.call("b200i_add", dev.index, _stream(dev), _vp(out), _vp(a), _vp(b), a.numel())
    return out


class TransformerBlock(object):
    #: the profile this build computes in; a block asked for another one is refused
    NUMERIC_PROFILE = "mojolearn.identical.transformer.fp32.v1"

    _NAMES = {"q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "norm1": "input_layernorm.weight", "norm1_b": "input_layernorm.bias", "q": "q_proj.weight", "q_b": "q_proj.bias",
              "k": "k_proj.weight", "k_b": "k_proj.bias", "v": "v_proj.weight", "v_b": "v_proj.bias", "o": "o_proj.weight",
              "o_b": "o_proj.bias", "norm2": "post_attention_layernorm.weight", "norm2_b": "post_attention_layernorm.bias",
              "gate": "gate_proj.weight", "gate_b": "gate_proj.bias", "up": "up_proj.weight", "up_b": "up_proj.bias",
              "down": "down_proj.weight", "down_b": "down_proj.bias"}

    def __init__(self, weights, *, n_heads, n_kv_heads=None, head_dim=None, window=0, rope_theta=10000.0, rope_scaling=None,
                 rope_dim=None, max_positions=MAX_POSITIONS, qkv_bias=False, o_bias=False, norm="rmsnorm", norm_eps=1e-6,
                 norm_bias=False, mlp="swiglu", mlp_bias=False, qk_norm=False, attn_softcap=None, numeric_profile=None,
                 numeric_mode=None, rope=True, device=None):
        """The reference's constructor (python/mojolearn/_transformer_impl.py:408-419), option for option:
        `rope_scaling` None or a dict in the HuggingFace spelling ({"rope_type": "linear", "factor": f}, or "llama3"
        with low_freq_factor, high_freq_factor and original_max_position_embeddings); `rope_dim` the rotated columns
        of a head (partial rotary); `max_positions` the absolute-position ceiling the model declares; `qk_norm` an
        RMSNorm over each head's vector of q and k before the rotation (`q_norm.weight`, `k_norm.weight`, [head_dim]);
        `attn_softcap` caps every scaled score as cap * tanh(score / cap). `rope=False` and `device` are this
        package's own (learned positions are an extension; the reference's block always rotates)."""
        if numeric_mode not in (None, "identical"):
            raise RuntimeError("mojolearn_b200 has only the identical build")
        if numeric_profile not in (None, self.NUMERIC_PROFILE, "fp32", "float32"):
            raise ValueError("numeric_profile %r is not spelled by this build (it computes %s)" % (numeric_profile, self.NUMERIC_PROFILE))
        _native.require_device()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        if norm not in NORM_KINDS or mlp not in MLP_KINDS:
            raise ValueError("unknown norm %r or mlp %r" % (norm, mlp))
        if norm_bias and norm != "layernorm":
            raise ValueError("an RMSNorm carries no bias (norm_bias needs layernorm)")
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads or n_heads)
        self.window, self.rope, self.rope_theta = int(window or 0), bool(rope), float(rope_theta)
        self.rope_scaling = self._rope_scaling_fields(rope_scaling)
        self.max_positions = int(max_positions)
        if self.max_positions < 1:
            raise ValueError("max_positions must be positive")
        self.qk_norm = bool(qk_norm)
        if self.qk_norm and norm == "layernorm":
            raise ValueError("qk_norm is an RMSNorm over each head: it cannot follow a layernorm block REFUSED")
        self.attn_softcap = float(attn_softcap) if attn_softcap else 0.0
        if attn_softcap is not None and not (np.isfinite(float(attn_softcap)) and float(attn_softcap) > 0.0):
            raise ValueError("attn_softcap must be a finite positive float, got %r" % (attn_softcap,))
        self.norm_kind, self.norm_eps, self.norm_bias = NORM_KINDS[norm], float(norm_eps), bool(norm_bias)
        self.mlp_kind, self.mlp_bias, self.qkv_bias, self.o_bias = MLP_KINDS[mlp], bool(mlp_bias), bool(qkv_bias), bool(o_bias)
        self.weight_format = lowbit.format_of({k: v for k, v in weights.items() if lowbit.is_packed(v)})

        def vec(slot, need=True):
            name = self._NAMES[slot]
            if name not in weights:
                if need:
                    raise ValueError("weights lack %r" % name)
                return None
            return _vector(weights[name], name, self.device)

        def lin(slot, bias_slot, with_bias):
            name = self._NAMES[slot]
            if name not in weights:
                raise ValueError("weights lack %r" % name)
            bias = None
            if with_bias:
                bname = self._NAMES[bias_slot]
                if bname not in weights:
                    raise ValueError("weights lack %r" % bname)
                bias = weights[bname]
            return Linear(weights[name], self.device, bias)

        self.q_norm_w = vec("q_norm") if self.qk_norm else None
        self.k_norm_w = vec("k_norm") if self.qk_norm else None
        for slot in ("q_norm", "k_norm"):
            if not self.qk_norm and self._NAMES[slot] in weights:
                raise ValueError("weights carry %r but qk_norm is off REFUSED" % self._NAMES[slot])
        self.norm1_w, self.norm2_w = vec("norm1"), vec("norm2")
        self.norm1_b = vec("norm1_b") if self.norm_bias else None
        self.norm2_b = vec("norm2_b") if self.norm_bias else None
        self.q, self.k, self.v = (lin(s, s + "_b", self.qkv_bias) for s in ("q", "k", "v"))
        self.o = lin("o", "o_b", self.o_bias)
        self.gated = self.mlp_kind in GATED
        self.gate = lin("gate", "gate_b", self.mlp_bias) if self.gated else None
        self.up = lin("up", "up_b", self.mlp_bias)
        self.down = lin("down", "down_b", self.mlp_bias)
        self.d_model = self.q.in_features
        self.head_dim = int(head_dim or self.q.out_features // self.n_heads)
        if self.q.out_features != self.n_heads * self.head_dim or self.k.out_features != self.n_kv_heads * self.head_dim:
            raise ValueError("projection widths do not match n_heads * head_dim")
        if self.n_heads % self.n_kv_heads or self.head_dim % 2:
            raise ValueError("n_heads must be a multiple of n_kv_heads and head_dim even")
        self.rope_dim = int(rope_dim or self.head_dim)
        if self.rope_dim <= 0 or self.rope_dim > self.head_dim or self.rope_dim % 2:
            raise ValueError("transformer: the rotary table's rope_dim %d does not fit head_dim %d REFUSED" % (self.rope_dim, self.head_dim))
        if self.qk_norm and (tuple(self.q_norm_w.shape) != (self.head_dim,) or tuple(self.k_norm_w.shape) != (self.head_dim,)):
            raise ValueError("q_norm.weight and k_norm.weight must be (%d,)" % self.head_dim)
        self.inter = self.up.out_features
        # q|k|v and gate|up as one product each: fewer, wider launches, the same cells
        self.widths = (self.q.out_features, self.k.out_features, self.v.out_features)
        self.qkv = Linear.concat([self.q, self.k, self.v])
        if self.qkv is not None:
            self.q = self.k = self.v = None
        self.gateup = Linear.interleave(self.gate, self.up) if self.gated else None  # rows gate_0, up_0, gate_1, up_1, ...
        if self.gateup is not None:
            self.gate = self.up = None

        self.group, self.exchange, self.by_heads = None, None, False  # set by shard(): the process group this block is cut across, its peer exchange
        self.heads_local, self.kv_local, self.inter_local = self.n_heads, self.n_kv_heads, self.inter

    PROJECTIONS = ("qkv", "q", "k", "v", "o", "gateup", "gate", "up", "down")

    def shard(self, group, rank, world, exchange=None):
        """Cut the block across `world` ranks along bit-neutral axes only. With the head counts divisible by the
        world, a rank keeps its heads' rows of q, k, v (so rotary, the KV cache and the whole attention are local
        to the rank: a head never reads another head), gathers the context columns, keeps its rows of o, of gate
        and of up (the activation is elementwise, so it is local too), gathers the activation columns, and keeps
        its rows of down. Four all-gathers of finished float32 words per block, no k is ever split. Otherwise
        every projection is cut by output rows and gathered, and the seams between them run replicated.
        `exchange` (a `parallel.PeerExchange`) carries the gathers of calls it can take; the rest use the group."""
        if world == 1:
            return
        self.exchange = exchange
        by_heads = self.n_heads % world == 0 and self.n_kv_heads % world == 0 and self.inter % world == 0
        if not by_heads:
            for slot in self.PROJECTIONS:
                full = getattr(self, slot)
                if full is not None:
                    setattr(self, slot, ShardedLinear(full, group, rank, world, exchange))
            return
        hd = self.head_dim
        self.heads_local, self.kv_local = self.n_heads // world, self.n_kv_heads // world
        self.inter_local = self.inter // world
        wq, wk, wv = self.widths
        q0, k0 = rank * self.heads_local * hd, rank * self.kv_local * hd
        qn, kn = self.heads_local * hd, self.kv_local * hd
        if self.qkv is not None:
            parts = [self.qkv.shard_rows(q0, q0 + qn), self.qkv.shard_rows(wq + k0, wq + k0 + kn),
                     self.qkv.shard_rows(wq + wk + k0, wq + wk + k0 + kn)]
            self.qkv = Linear.concat(parts)
        else:
            self.q, self.k, self.v = self.q.shard_rows(q0, q0 + qn), self.k.shard_rows(k0, k0 + kn), self.v.shard_rows(k0, k0 + kn)
        self.widths = (qn, kn, kn)
        i0, i1 = rank * self.inter_local, (rank + 1) * self.inter_local
        if self.gateup is not None:
            self.gateup = self.gateup.shard_rows(2 * i0, 2 * i1)  # the interleaved rows of this rank's activation columns
        else:
            self.up = self.up.shard_rows(i0, i1)
            if self.gate is not None:
                self.gate = self.gate.shard_rows(i0, i1)
        self.o = ShardedLinear(self.o, group, rank, world, exchange)
        self.down = ShardedLinear(self.down, group, rank, world, exchange)
        self.group, self.by_heads = group, True

    def allocate_state(self, batch, max_tokens, window=None):
        return TransformerState(batch, self.kv_local, int(max_tokens), self.head_dim, self.device,
                                self.window if window is None else window)

    def decode_session(self, state):
        """Open a resident decode session on `state` (see TransformerDecodeSession)."""
        if state is None:
            raise ValueError("decode_session: a state is required")
        if state.session is not None and state.session.is_open:
            raise RuntimeError("decode_session: the state is already resident in an open session")
        if int(state.window) != int(self.window):
            raise ValueError("decode_session: the state was allocated for window %d, the block has window %d" %
                             (state.window, self.window))
        return TransformerDecodeSession(self, state)

    @staticmethod
    def _rope_scaling_fields(rope_scaling):
        """(kind, factor, low_freq_factor, high_freq_factor, original_max_positions): kind 0 none, 1 linear, 2 llama3."""
        if not rope_scaling:
            return (0, 1.0, 1.0, 4.0, 8192)
        kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
        if kind in (None, "default"):
            return (0, 1.0, 1.0, 4.0, 8192)
        if kind not in ("linear", "llama3"):
            raise ValueError("rope_scaling %r is not spelled (linear and llama3 are) REFUSED" % (kind,))
        if "factor" not in rope_scaling:
            raise ValueError("rope_scaling %r needs its factor" % (kind,))
        return ({"linear": 1, "llama3": 2}[kind], float(rope_scaling["factor"]), float(rope_scaling.get("low_freq_factor", 1.0)),
                float(rope_scaling.get("high_freq_factor", 4.0)), int(rope_scaling.get("original_max_position_embeddings", 8192)))

    def rope_tables(self, pos0, l, position=None):
        """cos and sin [l, rope_dim / 2] for this call's positions; the same for every block of a model."""
        dev, st = self.device, _stream(self.device)
        cosv = torch.empty((l, self.rope_dim // 2), dtype=torch.float32, device=dev)
        sinv = torch.empty_like(cosv)
        kind, factor, lo, hi, old = self.rope_scaling
        if kind == 0 and self.rope_dim == self.head_dim:  # the default record: the frozen v1 entry points
            if position is None:
                _native.call("b200i_rope_table", dev.index, st, _vp(cosv), _vp(sinv), pos0, l, self.head_dim, self.rope_theta)
            else:
                _native.call("b200i_rope_table_at", dev.index, st, _vp(cosv), _vp(sinv), _vp(position), l, self.head_dim,
                             self.rope_theta)
        else:
            _native.call("b200i_rope_table_opts", dev.index, st, _vp(cosv), _vp(sinv), pos0, _vp(position), l, self.rope_dim,
                         self.rope_theta, kind, factor, lo, hi, old)
        return cosv, sinv

    # -- the block on device tensors: x [B, L, d_model] -> [B, L, d_model]; state is advanced by L
    def forward_device(self, x, state, position=None, rope=None, delta=None, defer_add=False):
        """`position`, when given, is a device int32 word holding the tokens cached before this call: the
        position-dependent kernels read it instead of taking the host's count as an argument, so the launches
        can be captured in a CUDA graph and replayed at later positions (the host count still sizes and checks).
        `rope` = the (cos, sin) tables of this call when the caller has them (a model computes them once for all
        its blocks). `delta` [B*L, d_model] = a residual update of x not yet added: the add rides in the first
        norm's pass. With `defer_add` the block returns (r, d) with its output = r + d left to the next norm."""
        b, l, dm = x.shape
        if dm != self.d_model:
            raise ValueError("x has width %d, the block %d" % (dm, self.d_model))
        pos0, m = state.cached_tokens, b * l
        if pos0 + l > state.max_tokens:
            raise ValueError("transformer: this call would use %d KV slots and the cache holds %d REFUSED" %
                             (pos0 + l, state.max_tokens))
        ceiling = min(self.max_positions, MAX_POSITIONS * (int(self.rope_scaling[1]) if self.rope_scaling[0] == 1 else 1))
        if pos0 + l > ceiling:
            raise ValueError("transformer: absolute position %d is at or beyond %d" % (pos0 + l - 1, ceiling))
        dev, st = x.device, _stream(x.device)
        x2 = x.reshape(m, dm).contiguous()
        if delta is None:
            n1 = norm(x2, self.norm1_w, self.norm1_b, self.norm_eps, self.norm_kind)
        else:
            x2, n1 = add_norm(x2, delta, self.norm1_w, self.norm1_b, self.norm_eps, self.norm_kind)
        if self.qkv is not None:
            fused = self.qkv(n1)
            wq, wk, wv = self.widths
            q, k, v, ld = fused[:, :wq], fused[:, wq:wq + wk], fused[:, wq + wk:], fused.shape[1]
        else:
            q, k, v, ld = self.q(n1), self.k(n1), self.v(n1), 0
        if self.qk_norm:
            # an RMSNorm over each head's vector of q and of k, before the rotation (the plain form, or the offset form
            # when the block's norm is the offset form): rows of width head_dim with the shared [head_dim] weight
            kind = 2 if self.norm_kind == 2 else 0
            q = norm(q.contiguous().reshape(m * self.heads_local, self.head_dim), self.q_norm_w, None, self.norm_eps, kind).reshape(m, -1)
            k = norm(k.contiguous().reshape(m * self.kv_local, self.head_dim), self.k_norm_w, None, self.norm_eps, kind).reshape(m, -1)
            if ld:
                v, ld = v.contiguous(), 0
        cosv = sinv = None
        if self.rope:
            cosv, sinv = rope if rope is not None else self.rope_tables(pos0, l, position)
        cap = state.max_tokens
        used = pos0 + l
        qr = torch.empty((m, self.heads_local * self.head_dim), dtype=torch.float32, device=dev)
        ctx = torch.empty((m, self.heads_local * self.head_dim), dtype=torch.float32, device=dev)
        with _prof.span("rope_cache"):
            _native.call("b200i_qkv_rope_cache", dev.index, st, _vp(qr), _vp(state.k), _vp(state.v), _vp(q), _vp(k), _vp(v), ld,
                         _vp(cosv), _vp(sinv), b, l, self.heads_local, self.kv_local, self.head_dim, cap, pos0, _vp(position),
                         self.rope_dim)
        att = _prof.span("attention")
        att.__enter__()
        if position is None:
            s = used - (max(0, pos0 - (self.window - 1)) if self.window else 0)
            scores = torch.empty((_native.lib().b200i_attention_scratch_floats(b, l, self.heads_local, s),), dtype=torch.float32, device=dev)
            _native.call("b200i_attention", dev.index, st, _vp(ctx), _vp(qr), _vp(state.k), _vp(state.v), _vp(scores), b, l,
                         self.heads_local, self.kv_local, self.head_dim, cap, used, self.window, self.attn_softcap)
        else:
            s = min(cap, self.window - 1 + l) if self.window else cap  # the most keys any later position sees
            scores = torch.empty((_native.lib().b200i_attention_scratch_floats(b, l, self.heads_local, s),), dtype=torch.float32, device=dev)
            _native.call("b200i_attention_at", dev.index, st, _vp(ctx), _vp(qr), _vp(state.k), _vp(state.v), _vp(scores), b, l,
                         self.heads_local, self.kv_local, self.head_dim, cap, _vp(position), self.window, self.attn_softcap)
        att.__exit__()
        del scores
        if self.by_heads:
            with _prof.span("gather"):
                ctx = gather_columns(ctx, self.group, self.exchange)  # heads are rank-major, so the gathered columns are in head order
        r1, n2 = add_norm(x2, self.o(ctx), self.norm2_w, self.norm2_b, self.norm_eps, self.norm_kind)
        if not self.gated:
            # an ungated MLP's activation is elementwise on the up projection: it rides in that product's store
            # (mlp kinds 1, 2, 3 = gelu, gelu_tanh, silu are the store's activation codes)
            act = self.up(n2, act=self.mlp_kind)
        else:
            gu = self.gateup
            gathered = False
            if gu is not None and _native.lib().b200i_pair_epilogue_fits(m, gu.out_features, gu.in_features, OP_NT) and self.by_heads:
                # the same, sharded: the gather that follows folds the product's leaf groups and applies the gated store itself
                act, gathered = product_gather(gu, n2, {0: 4, 4: 5, 5: 6}[self.mlp_kind], self.group, self.exchange), True
            elif gu is not None and _native.lib().b200i_pair_epilogue_fits(m, gu.out_features, gu.in_features, OP_NT):
                # a decode-sized call: the gated activation rides in the store of the gate|up product (mlp kinds 0, 4,
                # 5 = swiglu, geglu, geglu_tanh are the store's pair codes 4, 5, 6)
                with _prof.span("product"):
                    act = torch_ops.product(n2, gu.w, gu.scale, gu.kind, OP_NT, bias=gu.bias, act={0: 4, 4: 5, 5: 6}[self.mlp_kind],
                                            out=torch.empty((m, self.inter_local), dtype=torch.float32, device=dev))
            else:
                act = torch.empty((m, self.inter_local), dtype=torch.float32, device=dev)
                if gu is not None:
                    fused = gu(n2)
                    with _prof.span("activation"):
                        _native.call("b200i_act_mul", dev.index, st, _vp(act), _vp(fused), None, m, self.inter_local, fused.shape[1],
                                     self.mlp_kind, 1)
                else:
                    up, gate = self.up(n2), self.gate(n2)
                    with _prof.span("activation"):
                        _native.call("b200i_act_mul", dev.index, st, _vp(act), _vp(gate), _vp(up), m, self.inter_local, 0, self.mlp_kind, 0)
        if self.by_heads and not gathered:
            with _prof.span("gather"):
                act = gather_columns(act, self.group, self.exchange)
        d = self.down(act)
        state.cached_tokens = used
        if defer_add:
            return r1.reshape(b, l, dm), d
        return add(r1, d).reshape(b, l, dm)

    def _run(self, x, state):
        host = not isinstance(x, torch.Tensor)
        if host:
            a = np.asarray(x)
            if a.dtype != np.float32:
                raise TypeError("x must be float32, got %s" % a.dtype)
            if not np.isfinite(a).all():
                raise ValueError("non-finite values in x REFUSED")
            xt = torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        else:
            xt = x
        if xt.dim() != 3:
            raise ValueError("x must be [B, L, d_model]")
        if state is None:
            state = self.allocate_state(xt.shape[0], xt.shape[1])
        y = self.forward_device(xt, state)
        if host:
            torch_ops.check_status(self.device)  # a host caller gets the answer or an error, never a partial answer
        return y.cpu().numpy() if host else y

    def forward(self, x, state=None, *, lengths=None):
        """`lengths` makes the batch ragged (reference `_transformer_impl.py:527-553`): B lengths in [1, L]; row i is real
        at positions [0, lengths[i]) and padding after. Each real position's output equals the row run alone at its own
        length and padding positions output exactly +0.0; whatever sits in the padding of x is never read. Not allowed
        together with a state. The rows are run one by one: a row's bits do not depend on its batch."""
        if lengths is None:
            return self._run(x, state)
        if state is not None:
            raise ValueError("lengths is not allowed together with a state")
        host = not isinstance(x, torch.Tensor)
        shape = tuple(np.asarray(x).shape) if host else tuple(x.shape)
        if len(shape) != 3:
            raise ValueError("x must be [B, L, d_model]")
        lens = [int(n) for n in lengths]
        if len(lens) != shape[0] or any(n < 1 or n > shape[1] for n in lens):
            raise ValueError("lengths must hold B values in [1, L]")
        if host:
            xa = np.asarray(x)
            out = np.zeros(shape, dtype=np.float32)
            for i, n in enumerate(lens):
                out[i, :n] = self._run(np.ascontiguousarray(xa[i:i + 1, :n]), None)[0]
            return out
        out = torch.zeros(shape, dtype=torch.float32, device=x.device)
        for i, n in enumerate(lens):
            out[i, :n] = self._run(x[i:i + 1, :n].contiguous(), None)[0]
        return out

    def step(self, x, state):
        """One decode step: x [B, 1, d_model] (or [B, d_model]) against the cached tokens."""
        if x.ndim == 2:
            return self._run(x[:, None, :], state)[:, 0, :]
        return self._run(x, state)

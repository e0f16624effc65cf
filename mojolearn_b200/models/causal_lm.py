"""`CausalLM`: embedding -> decoder blocks -> final norm -> lm_head, with prefill,
single-step decoding and greedy generation, device resident.

Mirrors python/mojolearn/models/causal_lm.py of the reference (:121-209:
`forward(ids, state)`, `step`, `allocate_state`, `generate(ids, max_new_tokens,
greedy=True)`; ids are `(batch, length)` int32, logits `(B, L, V)` float32;
greedy ties go to the lowest id, :190). The three non-block steps are the
reference's primitives: embedding gather `Y = ftz(W[id])`, the final norm, and
the head as a `gemm.fp32.v1` OP_NT product (bindings/_mojolearn_training.mojo
:575-587, :607-619, :683-696).

Weights use HuggingFace names (`model.embed_tokens.weight`,
`model.layers.N.self_attn.q_proj.weight`, ..., `model.norm.weight`,
`lm_head.weight`); 2-D projection weights may be `lowbit`-packed.

Extensions the reference does not have: learned absolute positions with
`positions="learned"` (`model.embed_positions.weight`, one plain add, rotary
off), a LayerNorm final norm, and output-column sharding across one process per
GPU: with a `torch.distributed` group every projection and the head keep only
their rows [r*N/g, (r+1)*N/g) and the full activation is rebuilt by an NCCL
all-gather. A cell reads one weight row and all of k, so the shard moves no bit:
the logits equal the single-GPU logits word for word.
"""
import copy
import ctypes
import os

import numpy as np
import torch

from .. import _native
from ..parallel import ExchangeUnavailable, PeerExchange, exchange_heads, gather_columns, shard_bounds
from ..transformer import Linear, ShardedLinear, TransformerBlock, TransformerState, _stream, _vector, _vp, add, add_norm, norm, NORM_KINDS


class CausalLMConfig(object):
    """The architecture of a decoder LM: what the reference's `ModelPlan` (python/mojolearn/models/config.py) carries
    for a transformer family: the shape and every block option."""

    def __init__(self, vocab, d_model, n_layers, n_heads, n_kv_heads=None, head_dim=None, intermediate=None, norm="rmsnorm",
                 norm_eps=1e-6, norm_bias=False, mlp="swiglu", mlp_bias=False, qkv_bias=False, o_bias=False,
                 positions="rope", rope_theta=10000.0, max_positions=8192, window=0, rope_scaling=None, rope_dim=None,
                 qk_norm=False, attn_softcap=None, tie_word_embeddings=False):
        self.vocab, self.d_model, self.n_layers, self.n_heads = vocab, d_model, n_layers, n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        self.head_dim = head_dim or d_model // n_heads
        self.intermediate = intermediate or 4 * d_model
        self.norm, self.norm_eps, self.norm_bias = norm, norm_eps, norm_bias
        self.mlp, self.mlp_bias, self.qkv_bias, self.o_bias = mlp, mlp_bias, qkv_bias, o_bias
        if positions not in ("rope", "learned"):
            raise ValueError("positions must be 'rope' or 'learned'")
        self.positions, self.rope_theta, self.max_positions, self.window = positions, rope_theta, max_positions, window
        self.rope_scaling, self.rope_dim, self.qk_norm, self.attn_softcap = rope_scaling, rope_dim, qk_norm, attn_softcap
        self.tie_word_embeddings = bool(tie_word_embeddings)


class CausalLMState(object):
    """One block state per layer, the batch size, the capacity and the tokens consumed."""

    def __init__(self, layers, batch_size, max_tokens):
        self.layers, self.batch_size, self.max_tokens = layers, batch_size, max_tokens

    @property
    def positions(self):
        return self.layers[0].cached_tokens if self.layers else 0


class CausalLM(object):
    #: rows (batch x new tokens) up to which a sharded model's gathers go through the peer exchange
    EXCHANGE_ROWS = 64

    def __init__(self, config, weights, *, weight_format="float32", max_positions=None, device=None, numeric_profile=None,
                 group=None, exchange=None, prefill_by_batch=True, emulate_world=0):
        """`group`: a torch.distributed group of one process per GPU; the model is then cut by output columns
        (see the module text). `exchange`: True / False forces or forbids the store-side peer exchange for the
        decode-step gathers (default: on, unless MOJOLEARN_B200_EXCHANGE=0). `prefill_by_batch`: a prompt on a
        fresh state is cut by SEQUENCES instead (each rank runs its share of the batch through the whole model,
        then the KV caches are re-cut to the decode layout by one all-to-all): the other bit-neutral axis.
        `emulate_world` (timing only): build rank 0's share of a model cut over that many ranks, with no process
        group and `parallel.LoopbackExchange` in place of the exchange; the outputs are then not the model's.
        `weight_format` ("float32", "bfloat16" or "int8"), `max_positions` and `numeric_profile` are the reference's
        keywords (python/mojolearn/models/causal_lm.py:126-131): float32 projection weights are packed into the asked
        storage format on the way in (weights that arrive packed keep their own), a smaller `max_positions` lowers
        the model's position ceiling, and a profile this build does not compute is refused."""
        _native.require_device()
        if weight_format not in ("float32", "bfloat16", "int8"):
            raise ValueError("weight_format must be 'float32', 'bfloat16' or 'int8', got %r" % (weight_format,))
        if numeric_profile not in (None, TransformerBlock.NUMERIC_PROFILE, "fp32", "float32"):
            raise ValueError("numeric_profile %r is not spelled by this build" % (numeric_profile,))
        if device == "auto":
            device = None
        self.weight_format = weight_format
        if weight_format != "float32":
            from .. import lowbit
            weights = {k: (lowbit.pack_one(np.asarray(v, dtype=np.float32), weight_format)
                           if (isinstance(v, np.ndarray) and v.ndim == 2 and v.dtype == np.float32 and "embed" not in k) else v)
                       for k, v in weights.items()}
        if max_positions is not None:
            config = copy.copy(config)
            config.max_positions = min(int(max_positions), config.max_positions)
        self.config = cfg = config
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.group, self.rank, self.world = group, 0, 1
        if group is not None:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

        def get(name):
            for key in (name, "model." + name):
                if key in weights:
                    return weights[key]
            raise ValueError("weights lack %r" % name)

        self.embed = _vector(get("embed_tokens.weight"), "embed_tokens.weight", self.device)
        if tuple(self.embed.shape) != (cfg.vocab, cfg.d_model):
            raise ValueError("embed_tokens.weight must be (%d, %d)" % (cfg.vocab, cfg.d_model))
        self.pos_table = None
        if cfg.positions == "learned":
            self.pos_table = _vector(get("embed_positions.weight"), "embed_positions.weight", self.device)
        self.blocks, self.full_blocks = [], []
        self.exchange = None
        if emulate_world and emulate_world > 1 and group is None:
            from ..parallel import LoopbackExchange
            self.world, self.exchange, prefill_by_batch = int(emulate_world), LoopbackExchange(emulate_world), False
        self.prefill_by_batch = bool(prefill_by_batch) and self.world > 1
        if self.world > 1 and self.exchange is None:
            want = exchange if exchange is not None else os.environ.get("MOJOLEARN_B200_EXCHANGE", "1") != "0"
            if want:
                rows = self.EXCHANGE_ROWS
                hd = cfg.head_dim
                per_block = rows * (cfg.n_heads * hd + 2 * cfg.d_model + cfg.intermediate) + 4 * 64  # words of a block's four gathers
                try:
                    self.exchange = PeerExchange(group, self.device, rows, max(cfg.vocab, cfg.intermediate, cfg.d_model, cfg.n_heads * hd),
                                                 cfg.n_layers * per_block + rows * cfg.vocab + 64)
                except ExchangeUnavailable:  # raised by every rank together: the gathers go through NCCL
                    self.exchange = None
        for i in range(cfg.n_layers):
            bw = {}
            for key, val in weights.items():
                for prefix in ("model.layers.%d." % i, "layers.%d." % i):
                    if key.startswith(prefix):
                        bw[key[len(prefix):].replace("self_attn.", "").replace("mlp.", "")] = val
            blk = TransformerBlock(bw, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, window=cfg.window,
                                   rope=cfg.positions == "rope", rope_theta=cfg.rope_theta, rope_scaling=cfg.rope_scaling,
                                   rope_dim=cfg.rope_dim, max_positions=cfg.max_positions, qkv_bias=cfg.qkv_bias,
                                   o_bias=cfg.o_bias, norm=cfg.norm, norm_eps=cfg.norm_eps, norm_bias=cfg.norm_bias, mlp=cfg.mlp,
                                   mlp_bias=cfg.mlp_bias, qk_norm=cfg.qk_norm, attn_softcap=cfg.attn_softcap, device=self.device)
            self.full_blocks.append(blk)
            if self.world > 1:
                blk = copy.copy(blk)  # the shards are row views of the same weights; only the fused q|k|v and gate|up shards are copies
                blk.shard(group, self.rank, self.world, self.exchange)
            self.blocks.append(blk)
        self.final_w = _vector(get("norm.weight"), "norm.weight", self.device)
        self.final_b = _vector(get("norm.bias"), "norm.bias", self.device) if cfg.norm_bias else None
        head = weights.get("lm_head.weight", None)
        self.head = Linear(head if head is not None else self.embed, self.device)
        if self.head.out_features != cfg.vocab:
            raise ValueError("lm_head.weight must have %d rows" % cfg.vocab)
        self.full_head = self.head
        if self.world > 1:
            self.head = ShardedLinear(self.head, group, self.rank, self.world, self.exchange)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)

    @classmethod
    def load(cls, path, *, weight_format="float32", max_positions=None, device=None, numeric_profile=None, **kw):
        """A checkpoint directory: `config.json` plus `model.safetensors`, or `model.safetensors.index.json` and its
        shards (reference python/mojolearn/models/causal_lm.py:139-150). The config is mapped family by family
        (`models.config.plan_for`; a field the blocks cannot honor is refused by name), the tensors are read exactly
        (BF16 and F16 checkpoints widen exactly to float32; with weight_format "bfloat16" BF16 matrices stay as their
        bits), and a tensor the plan needs and the checkpoint lacks is refused by name."""
        from . import config as _config, safetensors as _safetensors
        plan = _config.plan_for(_config.read_config(path))
        weights = {}
        with _safetensors.Checkpoint.open(path) as ckpt:
            for name in _config.checkpoint_names(plan):
                if name not in ckpt:
                    raise ValueError("the checkpoint lacks %r, which a %d-layer model of this family needs" % (name, plan.n_layers))
                keep_bits = weight_format == "bfloat16" and name.endswith("_proj.weight") or (weight_format == "bfloat16" and name == "lm_head.weight")
                weights[name] = ckpt.read(name, bf16="bits" if keep_bits else "widen")
        return cls(plan, weights, weight_format=weight_format, max_positions=max_positions, device=device,
                   numeric_profile=numeric_profile, **kw)

    def allocate_state(self, batch_size, max_tokens):
        return CausalLMState([b.allocate_state(batch_size, max_tokens) for b in self.blocks], batch_size, int(max_tokens))

    def reset_state(self, state):
        """Empty the caches of `state`, keeping its batch size and capacity (reference causal_lm.py:177)."""
        for layer in state.layers:
            layer.cached_tokens = 0
            layer.session = None
        return state

    def parameters(self):
        """The model's tensors by checkpoint name, as they live on the device (packed weights as (storage, scale))."""
        out = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_w, "lm_head.weight": self.full_head.w}
        for i, blk in enumerate(self.full_blocks):
            for slot, name in blk._NAMES.items():
                for holder in (getattr(blk, slot, None), getattr(blk, slot + "_w", None)):
                    if isinstance(holder, torch.Tensor):
                        out["model.layers.%d.%s" % (i, name)] = holder
                    elif isinstance(holder, Linear):
                        out["model.layers.%d.%s" % (i, name)] = holder.w if holder.scale is None else (holder.w, holder.scale)
        return out

    def stream(self, ids, max_new_tokens, greedy=True):
        """A continuation stream (reference causal_lm.py:211): `read(n)` returns at most n new ids per row, (B, <= n)
        int32 on the host, and an empty (B, 0) array once `max_new_tokens` have been read."""
        if not greedy:
            raise ValueError("only greedy decoding is spelled")
        return _Stream(self, ids, int(max_new_tokens))

    def _ids(self, ids):
        if isinstance(ids, torch.Tensor):
            t = ids.to(self.device, torch.int32)
        else:
            a = np.asarray(ids)
            if a.dtype.kind not in "iu":
                raise TypeError("token ids must be integers")
            t = torch.from_numpy(np.ascontiguousarray(a.astype(np.int32))).to(self.device)
        if t.dim() != 2:
            raise ValueError("token ids must be (batch, length)")
        return t.contiguous()

    def hidden_device(self, ids, state, position=None, blocks=None):
        """Final-normed hidden states [B*L, d_model] for the ids, advancing the state. `position`: see
        TransformerBlock.forward_device. `blocks`: the unsharded blocks, for a prompt cut by sequences."""
        blocks = self.blocks if blocks is None else blocks
        if self.exchange is not None and blocks is self.blocks:
            self.exchange.begin_step()
        b, l = ids.shape
        dev, st, cfg = self.device, _stream(self.device), self.config
        if state.positions + l > cfg.max_positions:
            raise ValueError("absolute position %d is at or beyond max_positions %d" % (state.positions + l - 1, cfg.max_positions))
        x = torch.empty((b * l, cfg.d_model), dtype=torch.float32, device=dev)
        _native.call("b200i_embedding", dev.index, st, _vp(x), _vp(self.embed), _vp(ids), b * l, cfg.vocab, cfg.d_model,
                     _vp(self._status))
        if self.pos_table is not None:
            if state.positions + l > self.pos_table.shape[0]:
                raise ValueError("position table of %d rows is too short" % self.pos_table.shape[0])
            if position is None:
                _native.call("b200i_add_positions", dev.index, st, _vp(x), _vp(self.pos_table), b * l, l, state.positions,
                             cfg.d_model)
            else:
                _native.call("b200i_add_positions_at", dev.index, st, _vp(x), _vp(self.pos_table), b * l, l, _vp(position),
                             cfg.d_model)
        h, delta = x.reshape(b, l, cfg.d_model), None
        rope = None  # one rotary table per call: every block is at the same positions
        if blocks and blocks[0].rope:
            rope = blocks[0].rope_tables(state.positions, l, position)
        for blk, bs in zip(blocks, state.layers):
            h, delta = blk.forward_device(h, bs, position, rope, delta, defer_add=True)  # each block's last add rides in the next norm
        h2 = h.reshape(b * l, cfg.d_model)
        if delta is None:
            return norm(h2, self.final_w, self.final_b, cfg.norm_eps, NORM_KINDS[cfg.norm])
        return add_norm(h2, delta, self.final_w, self.final_b, cfg.norm_eps, NORM_KINDS[cfg.norm])[1]

    def check_ids(self):
        """Raise if any id given since the last check was outside the vocabulary (reads one device word)."""
        if int(self._status.item()) != 0:
            self._status.zero_()
            raise ValueError("a token id is outside the embedding table")

    def check_status(self):
        """Raise if a bounded device-side wait ran out since the last check (synchronises the device)."""
        from .. import torch_ops
        torch_ops.check_status(self.device)

    def _prefill_by_batch(self, ids, state, last_only):
        """A prompt on a fresh state, cut by sequences: this rank runs rows [r*B/g, (r+1)*B/g) through the WHOLE model
        (a sequence's bits do not depend on its batch), the logits are all-gathered in rank = batch order, and every
        layer's keys and values move to the decode layout (this rank's heads of every sequence) by one all-to-all."""
        import torch.distributed as dist
        b, l = ids.shape
        bl, cfg = b // self.world, self.config
        mine = ids[self.rank * bl:(self.rank + 1) * bl].contiguous()
        local = CausalLMState([blk.allocate_state(bl, l) for blk in self.full_blocks], bl, l)
        hn = self.hidden_device(mine, local, None, self.full_blocks)
        if last_only:
            hn = hn.reshape(bl, l, -1)[:, -1, :].contiguous()
        part = self.full_head(hn)
        logits = torch.empty((self.world * part.shape[0], cfg.vocab), dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(logits, part.contiguous(), group=self.group)
        for src, dst, blk in zip(local.layers, state.layers, self.blocks):
            for a, z in ((src.k, dst.k), (src.v, dst.v)):
                if blk.kv_local != blk.n_kv_heads:   # decode keeps this rank's heads of every sequence
                    z[:, :, :l, :] = exchange_heads(a[:, :, :l, :], self.world, self.group)
                else:                                # decode keeps every head (the block is cut by rows only)
                    whole = torch.empty((b,) + tuple(a.shape[1:]), dtype=torch.float32, device=self.device)
                    dist.all_gather_into_tensor(whole, a.contiguous(), group=self.group)
                    z[:, :, :l, :] = whole[:, :, :l, :]
            dst.cached_tokens = l
            src.k = src.v = None
        return logits if last_only else logits.reshape(b, l, cfg.vocab)

    def forward_device(self, ids, state=None, last_only=False, position=None):
        ids = self._ids(ids)
        b, l = ids.shape
        if state is None:
            state = self.allocate_state(b, l)
        if self.prefill_by_batch and position is None and state.positions == 0 and l > 1 and b % self.world == 0 and b >= self.world:
            return self._prefill_by_batch(ids, state, last_only)
        hn = self.hidden_device(ids, state, position)
        if last_only:
            hn = hn.reshape(b, l, -1)[:, -1, :].contiguous()
            return self.head(hn)
        return self.head(hn).reshape(b, l, self.config.vocab)

    def forward(self, ids, state=None):
        """Logits (B, L, V) for the ids; with a state, appends to its caches."""
        host = not isinstance(ids, torch.Tensor)
        out = self.forward_device(ids, state)
        self.check_ids()
        if host:
            self.check_status()
        return out.cpu().numpy() if host else out

    def step(self, ids, state):
        """Logits (B, V) for one new token per row."""
        host = not isinstance(ids, torch.Tensor)
        t = self._ids(ids if (isinstance(ids, torch.Tensor) and ids.dim() == 2) or np.ndim(ids) == 2 else np.asarray(ids)[:, None])
        out = self.forward_device(t, state)[:, -1, :]
        self.check_ids()
        if host:
            self.check_status()
        return out.cpu().numpy() if host else out

    def argmax_device(self, logits2d):
        out = torch.empty((logits2d.shape[0],), dtype=torch.int32, device=logits2d.device)
        _native.call("b200i_argmax", logits2d.device.index, _stream(logits2d.device), _vp(out), _vp(logits2d.contiguous()),
                     logits2d.shape[0], logits2d.shape[1])
        return out

    def decode_session(self, state, logits, graph=True):
        """A resident greedy decode session over a prefilled state and the logits of its last position."""
        return DecodeSession(self, state, logits, graph)

    def generate(self, ids, max_new_tokens, greedy=True, state=None, return_logits=False, graph=True):
        """Prefill on `ids` (B, L), then `max_new_tokens` greedy steps; returns (B, L + new) ids. The whole
        continuation stays on the device: one host read at the end. With `graph` the decode step is captured
        once as a CUDA graph and replayed (same kernels, same bits, no per-launch host cost)."""
        if not greedy:
            raise ValueError("only greedy decoding is spelled")
        host = not isinstance(ids, torch.Tensor)
        t = self._ids(ids)
        b, l = t.shape
        if state is None:
            state = self.allocate_state(b, l + max_new_tokens)
        logits = self.forward_device(t, state, last_only=True)
        out, kept = [t], []
        session = DecodeSession(self, state, logits, graph)
        for step in range(max_new_tokens):
            out.append(session.next_ids().clone())
            if return_logits:
                kept.append(session.logits.clone())
            if step + 1 < max_new_tokens:
                session.step()
        self.check_ids()
        self.check_status()  # once per call, not per step
        seq = torch.cat(out, dim=1)
        seq = seq.cpu().numpy() if host else seq
        if return_logits:
            stack = torch.stack(kept, dim=1)
            return seq, (stack.cpu().numpy() if host else stack)
        return seq


class _Stream(object):
    def __init__(self, lm, ids, budget):
        t = lm._ids(ids)
        self.lm, self.left, self.batch = lm, budget, t.shape[0]
        self.state = lm.allocate_state(t.shape[0], t.shape[1] + budget)
        self.session = lm.decode_session(self.state, lm.forward_device(t, self.state, last_only=True))
        self.first = True

    def read(self, n):
        take = max(0, min(int(n), self.left))
        out = []
        for _ in range(take):
            if not self.first:
                self.session.step()
            self.first = False
            out.append(self.session.next_ids().clone())
        self.left -= take
        self.lm.check_ids()
        if not out:
            return np.zeros((self.batch, 0), dtype=np.int32)
        return torch.cat(out, dim=1).cpu().numpy()


class DecodeSession(object):
    """Greedy decoding with everything resident on the device (the reference's resident decode session,
    python/mojolearn/models/causal_lm.py:197-201).

    `next_ids()` is the argmax of the current logits, `step()` feeds it back: embedding, every block, the final
    norm, the head. The first step runs launch by launch; from the second on the step is captured once as a
    CUDA graph (the position lives in a device word that the graph itself advances) and replayed, which removes
    the host cost of its several hundred launches. Kernels and bits are those of `CausalLM.step`."""

    def __init__(self, lm, state, logits, graph=True):
        self.lm, self.state, self.use_graph = lm, state, bool(graph)
        self.logits = logits.contiguous()
        b = self.logits.shape[0]
        self.ids = torch.empty((b, 1), dtype=torch.int32, device=lm.device)
        self.position = torch.zeros(1, dtype=torch.int32, device=lm.device)
        self.graph, self.steps, self._fresh = None, 0, False
        self.graph_launches, self.replays = 0, 0  # kernels in the captured step; times it was replayed

    def check_status(self):
        """Raise if a bounded device-side wait ran out in any step so far (synchronises the device)."""
        self.lm.check_status()

    def next_ids(self):
        """(B, 1) int32 on the device: the greedy choice from the current logits."""
        if not self._fresh:
            self.ids.copy_(self.lm.argmax_device(self.logits).reshape(-1, 1))
            self._fresh = True
        return self.ids

    def _check_room(self):
        pos, cfg = self.state.positions, self.lm.config
        if pos + 1 > self.state.max_tokens:
            raise ValueError("transformer: this call would use %d KV slots and the cache holds %d REFUSED" %
                             (pos + 1, self.state.max_tokens))
        if pos + 1 > cfg.max_positions:
            raise ValueError("absolute position %d is at or beyond max_positions %d" % (pos, cfg.max_positions))

    def _captured_step(self):
        lm, dev = self.lm, self.lm.device
        out = lm.forward_device(self.ids, self.state, last_only=True, position=self.position)
        self.ids.copy_(lm.argmax_device(out).reshape(-1, 1))
        _native.call("b200i_advance_position", dev.index, _stream(dev), _vp(self.position), 1)
        return out

    def step(self):
        """Consume next_ids(); afterwards `logits` are those of the new position."""
        self.next_ids()
        self._check_room()
        if not self.use_graph or self.steps == 0:
            self.logits = self.lm.forward_device(self.ids, self.state, last_only=True)
            self._fresh = False
        else:
            if self.graph is None:
                self.position.fill_(self.state.positions)
                before = [s.cached_tokens for s in self.state.layers]
                torch.cuda.synchronize(self.lm.device)
                self.graph = torch.cuda.CUDAGraph()
                counted = _native.lib().b200i_launch_count()
                with torch.cuda.graph(self.graph):
                    self._out = self._captured_step()
                self.graph_launches = int(_native.lib().b200i_launch_count() - counted)
                for s, n in zip(self.state.layers, before):  # capturing launched nothing
                    s.cached_tokens = n
                if self.lm.group is not None and self.lm.world > 1:  # capture takes the ranks different times: start the replays together
                    import torch.distributed as dist
                    torch.cuda.synchronize(self.lm.device)
                    dist.barrier(self.lm.group)
            self.graph.replay()
            self.replays += 1
            for s in self.state.layers:
                s.cached_tokens += 1
            self.logits = self._out
            self._fresh = True  # the graph already wrote the next ids
        self.steps += 1
        return self.logits

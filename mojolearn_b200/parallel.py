"""Bit-neutral sharding of a linear layer across one process per GPU.

A cell C[i, j] of the identical-mode product reads row i of the activations and
row j of the weight and nothing else, and its bits depend on k and the profile
alone (reference gemm/IDENTICAL_FP32_CONTRACT.md:112-116). So the only axes a
layer may be cut along are output columns (weight rows) and batch; k is never
split and nothing is ever all-reduced, because a k split is a summation order.
Rank r keeps weight rows [r*N/g, (r+1)*N/g), computes its column slice with the
full k, and the slices are concatenated by an all-gather, which moves finished
float32 words and performs no arithmetic. The reference's own multi-device rule
is the same: byte copies only, never a collective that picks an order
(training/byte_lm_parallel.py:2-8, core/multi_gpu.mojo:2-6).
"""
import ctypes
import os

import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """Rows [lo, hi) of an n-row weight owned by `rank`; n must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d outside a world of %d" % (rank, world))
    if n % world:
        raise ValueError("%d output columns do not divide over %d ranks" % (n, world))
    return rank * n // world, (rank + 1) * n // world


def gather_columns(part, group=None, exchange=None):
    """[m, n/g] column slices on every rank -> the full [m, n] on every rank (rank order = column order). With a
    `PeerExchange` that takes the slice the ranks store their slices straight into each other's gathered matrix
    (one small kernel, no layout copy); otherwise an all-gather of the process group and a rank-major to
    column-major copy."""
    if exchange is not None and exchange.takes(part):
        return exchange.gather(part)
    world = dist.get_world_size(group)
    if world == 1:
        return part
    part = part.contiguous()
    m, w = part.shape
    gathered = torch.empty((world * m, w), dtype=part.dtype, device=part.device)  # rank-major concatenation
    dist.all_gather_into_tensor(gathered, part, group=group)
    return gathered.view(world, m, w).permute(1, 0, 2).reshape(m, world * w).contiguous()


class ExchangePlan(object):
    """Where the receive areas of a step's gathers live in an exchange buffer (host arithmetic only).

    A gather of [m, w] slices needs m * w * world pairs of 8 bytes in every rank's buffer. The first gather of a
    step lives alone in [0, first_zone): the next step's first gather may be written by a fast rank while a slow
    rank still reads this step's last area, so those two must never overlap; every later gather is bump-allocated
    behind that zone and the cursor returns there at `begin_step()`. Every rank runs the same sequence of calls,
    so every rank computes the same offsets."""

    ALIGN = 256

    def __init__(self, world, first_zone, total_bytes):
        self.world, self.first_zone, self.total_bytes = int(world), int(first_zone), int(total_bytes)
        self.site, self.cursor = 0, self.first_zone

    def needs_closing_gather(self):
        """True when the step so far has exactly one gather: the caller must add a second one (of anything) before the
        next step begins, because only a later gather of the same step orders the reuse of the first one's area."""
        return self.site == 1

    def begin_step(self):
        if self.site == 1:
            raise RuntimeError("a step with a single gather cannot use the peer exchange (two gathers order the reuse of the areas)")
        self.site, self.cursor = 0, self.first_zone

    def size(self, m, w):
        return (m * w * self.world * 8 + self.ALIGN - 1) // self.ALIGN * self.ALIGN

    def fits(self, m, w):
        size = self.size(m, w)
        return size <= self.first_zone if self.site == 0 else self.cursor + size <= self.total_bytes

    def place(self, m, w):
        """(index of the gather in its step, byte offset of its receive areas), advancing the plan."""
        if not self.fits(m, w):
            raise ValueError("the gather's receive areas do not fit the exchange")
        site, offset = self.site, (0 if self.site == 0 else self.cursor)
        if site > 0:
            self.cursor += self.size(m, w)
        self.site += 1
        return site, offset


class ExchangeUnavailable(RuntimeError):
    """Raised by every rank together when the peer exchange cannot be set up on some rank."""


class PeerExchange(object):
    """This rank's end of the store-side exchange of the CUDA library (`b200i_comm_*`): a buffer every rank of the
    node maps, into which the owners of column slices store their words. One object per model; `begin_step()` at
    the start of every model step, then `gather()` in the same order on every rank. A slice it cannot take (more
    rows than it was sized for, or the step's areas are used up) goes through the process group instead, which is
    always correct."""

    def __init__(self, group, device, max_rows, max_width, step_words):
        """`max_width`: the widest gathered matrix of a step's FIRST gather; `step_words`: float32 words of all the
        other gathered matrices of one step at `max_rows` rows."""
        from . import _native
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.max_rows = int(max_rows)
        first_zone = (self.max_rows * int(max_width) * 8 + 255) // 256 * 256
        self.total_bytes = first_zone + (int(step_words) * 8 + 255) // 256 * 256
        self.plan = ExchangePlan(self.world, first_zone, self.total_bytes)
        self._native = _native
        # Every rank takes every collective below whatever happens to it, and the ranks agree at the end whether the
        # exchange stands: a rank that cannot create or map a buffer (no peer access, no IPC) must not leave the others
        # waiting, and all of them then raise ExchangeUnavailable together (the caller falls back to NCCL gathers).
        comm, ok = ctypes.c_void_p(), 1
        handle = ctypes.create_string_buffer(64)
        try:
            if os.environ.get("MOJOLEARN_B200_EXCHANGE_FAIL_RANK") == str(self.rank):  # failure injection for the tests, on the host
                raise RuntimeError("injected exchange set-up failure")
            _native.call("b200i_comm_create", self.device.index, self.rank, self.world, self.total_bytes, ctypes.byref(comm))
            _native.call("b200i_comm_export", comm, ctypes.cast(handle, ctypes.c_void_p), 64)
        except Exception:  # noqa: BLE001
            ok = 0
        self.comm = comm
        mine = torch.tensor(list(handle.raw) + [ok], dtype=torch.uint8, device=self.device)
        everyone = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(everyone, mine, group=group)
        rows = [bytes(h.cpu().tolist()) for h in everyone]
        ok = int(all(r[64] == 1 for r in rows))
        if ok:
            try:
                for peer, raw in enumerate(rows):
                    if peer != self.rank:
                        _native.call("b200i_comm_attach", comm, peer, ctypes.cast(ctypes.create_string_buffer(raw[:64], 64), ctypes.c_void_p))
                torch.cuda.synchronize(self.device)
            except Exception:  # noqa: BLE001
                ok = 0
        agreed = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)  # also the barrier: every rank has zeroed its buffer and mapped every peer before anyone sends
        if int(agreed.item()) != 1:
            if comm:
                try:
                    _native.lib().b200i_comm_destroy(comm)
                except Exception:  # noqa: BLE001
                    pass
            self.comm = None
            raise ExchangeUnavailable("a rank could not create or map the peer exchange buffers")
        self._token = None

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def begin_step(self):
        if self.plan.needs_closing_gather():
            # the step that just ended gathered once (a long prompt whose only small gather was the head's): give it a
            # second, two-word gather so that the reuse of the first area stays ordered
            if self._token is None:
                self._token = torch.zeros((1, 2), dtype=torch.float32, device=self.device)
            self.gather(self._token)
        self.plan.begin_step()
        self._native.call("b200i_comm_advance", self.comm, self._stream())

    def takes(self, part):
        if part.dim() != 2 or part.dtype != torch.float32 or part.stride(1) != 1 or part.shape[0] > self.max_rows:
            return False
        return self.plan.fits(part.shape[0], part.shape[1])

    def gather(self, part, mode=0):
        m, w = part.shape
        _, offset = self.plan.place(m, w)
        out = torch.empty((m, self.world * w), dtype=torch.float32, device=self.device)
        self._native.call("b200i_comm_gather", self.comm, self._stream(), mode, offset, ctypes.c_void_p(out.data_ptr()), 0,
                          ctypes.c_void_p(part.data_ptr()), m, w, part.stride(0))
        return out

    def takes_shape(self, m, w):
        """Whether a finished slice of m rows and w columns can go through this exchange (`takes` before the slice exists)."""
        return m <= self.max_rows and self.plan.fits(m, w)

    def gather_nodes(self, ws, nodes, m, n, bias, act, mode=0):
        """`gather` for a slice `torch_ops.product_nodes` left as leaf-group nodes: fold, store epilogue, send and
        receive in one launch (`b200i_comm_gather_nodes`)."""
        w = n // 2 if act >= 4 else n
        _, offset = self.plan.place(m, w)
        out = torch.empty((m, self.world * w), dtype=torch.float32, device=self.device)
        self._native.call("b200i_comm_gather_nodes", self.comm, self._stream(), mode, offset, ctypes.c_void_p(out.data_ptr()), 0,
                          ctypes.c_void_p(ws.data_ptr()), nodes, m, n, ctypes.c_void_p(bias.data_ptr()) if bias is not None else None, act)
        return out

    def close(self):
        if self.comm is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self._native.lib().b200i_comm_destroy(self.comm)
            self.comm = None


class LoopbackExchange(object):
    """A stand-in exchange for TIMING one rank's share of a sharded step on a single GPU, with no other rank: a
    "gather" repeats the local slice `world` times, so every shape, launch and byte count is the real rank's but the
    values are not the model's. Used by `serve_bench --emulate-world` to separate a sharded step's own kernels from
    its communication; never by the model proper."""

    def __init__(self, world):
        self.world, self.rank = int(world), 0
        self._comm = None

    def takes_shape(self, m, w):
        return m * w * 8 <= 16 << 20

    def gather_nodes(self, ws, nodes, m, n, bias, act, mode=0):
        """The fold-and-send launch of the real exchange with nobody to send to: this rank's columns of the gathered
        matrix are the model's, the others are left as allocated."""
        from . import _native
        if self._comm is None:
            self._comm = ctypes.c_void_p()
            _native.call("b200i_comm_create", ws.device.index, 0, 1, 16 << 20, ctypes.byref(self._comm))
        w = n // 2 if act >= 4 else n
        out = torch.empty((m, self.world * w), dtype=torch.float32, device=ws.device)
        _native.call("b200i_comm_gather_nodes", self._comm, ctypes.c_void_p(torch.cuda.current_stream(ws.device).cuda_stream), mode, 0,
                     ctypes.c_void_p(out.data_ptr()), out.stride(0), ctypes.c_void_p(ws.data_ptr()), nodes, m, n,
                     ctypes.c_void_p(bias.data_ptr()) if bias is not None else None, act)
        return out

    def begin_step(self):
        pass

    def takes(self, part):
        return True

    def gather(self, part, mode=0):
        return part.repeat(1, self.world)


def exchange_heads(cache_rows, world, group=None):
    """Re-cut KV caches from batch shards to head shards. `cache_rows` is this rank's [b/g, heads, length, head_dim]
    (all heads of its own sequences); the result is [b, heads/g, length, head_dim] (this rank's heads of every
    sequence, sequences in rank order). One all-to-all of finished words: a copy, no arithmetic."""
    bl, heads, length, hd = cache_rows.shape
    hl = heads // world
    send = cache_rows.reshape(bl, world, hl, length, hd).permute(1, 0, 2, 3, 4).contiguous()  # [dest, b/g, heads/g, L, hd]
    recv = torch.empty_like(send)                                                              # [src,  b/g, heads/g, L, hd]
    dist.all_to_all_single(recv, send, group=group)
    return recv.reshape(world * bl, hl, length, hd)

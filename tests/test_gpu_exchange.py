"""The store-side exchange kernel (b200i_comm_gather) on ONE device.

A real exchange needs one process per GPU (tests/test_gpu_multi.py). Here its addressing, tags and epochs are checked
without any launch that waits for a later launch: with a world of one the rank receives nothing, and a world of two is
emulated by two exchange objects on the same device whose launches sit on one stream in an order in which every
awaited word has already been sent (rank 0 sends, rank 1 sends and receives, rank 0 receives).
"""
import ctypes

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native  # noqa: E402

SEND_RECV, SEND, RECV = 0, 1, 2


def _create(rank, world, nbytes):
    comm = ctypes.c_void_p()
    _native.call("b200i_comm_create", 0, rank, world, nbytes, ctypes.byref(comm))
    return comm


def _gather(comm, mode, area, out, part):
    m, w = out.shape[0], out.shape[1] // (2 if part is None else out.shape[1] // part.shape[1])
    ptr = ctypes.c_void_p(part.data_ptr()) if part is not None else None
    ld = part.stride(0) if part is not None else 0
    _native.call("b200i_comm_gather", comm, None, mode, area, ctypes.c_void_p(out.data_ptr()), out.stride(0), ptr, m, w, ld)


def test_world_of_one_copies_the_slice():
    comm = _create(0, 1, 1 << 20)
    g = torch.Generator(device="cuda").manual_seed(0)
    for epoch in range(3):
        _native.call("b200i_comm_advance", comm, None)
        for site, (m, w) in enumerate(((5, 12), (7, 13), (32, 2048))):  # paired and single-word widths
            part = torch.randn((m, w), generator=g, device="cuda")
            out = torch.full((m, w), -1.0, device="cuda")
            _gather(comm, SEND_RECV, site * 256 * 1024, out, part)
            torch.cuda.synchronize()
            assert torch.equal(out, part), (epoch, site)
    wide = torch.randn((4, 64), generator=g, device="cuda")
    out = torch.empty((4, 32), device="cuda")
    _gather(comm, SEND_RECV, 0, out, wide[:, 8:40])  # a column block of a wider matrix: the row pitch is honoured
    torch.cuda.synchronize()
    assert torch.equal(out, wide[:, 8:40])
    assert _native.lib().b200i_decode_status(0) == 0
    with pytest.raises(_native.NativeError, match="do not fit"):
        _gather(comm, SEND_RECV, 1 << 20, out, wide[:, 8:40])
    _native.lib().b200i_comm_destroy(comm)


def test_two_ranks_emulated_on_one_stream():
    c0, c1 = _create(0, 2, 2 << 20), _create(1, 2, 2 << 20)
    _native.call("b200i_comm_attach_local", c0, 1, c1)
    _native.call("b200i_comm_attach_local", c1, 0, c0)
    g = torch.Generator(device="cuda").manual_seed(1)
    for epoch in range(4):
        _native.call("b200i_comm_advance", c0, None)
        _native.call("b200i_comm_advance", c1, None)
        for site, (m, w) in enumerate(((3, 8), (32, 1024), (5, 7))):
            p0 = torch.randn((m, w), generator=g, device="cuda")
            p1 = torch.randn((m, w), generator=g, device="cuda")
            o0 = torch.full((m, 2 * w), -1.0, device="cuda")
            o1 = torch.full((m, 2 * w), -1.0, device="cuda")
            area = site * 640 * 1024
            _gather(c0, SEND, area, o0, p0)        # rank 0 sends (and places its own slice)
            _gather(c1, SEND_RECV, area, o1, p1)   # rank 1 sends, and finds rank 0's words already there
            _gather(c0, RECV, area, o0, None)      # rank 0 finds rank 1's
            torch.cuda.synchronize()
            want = torch.cat([p0, p1], dim=1)
            assert torch.equal(o0, want) and torch.equal(o1, want), (epoch, site)
    assert _native.lib().b200i_decode_status(0) == 0
    _native.lib().b200i_comm_destroy(c0)
    _native.lib().b200i_comm_destroy(c1)


def _nodes_product(x, w, scale, kind, bias, act):
    from mojolearn_b200 import torch_ops
    return torch_ops.product_nodes(x, w, scale, kind, bias=bias, act=act)


def _gather_nodes(comm, mode, area, out, ws, nodes, m, n, bias, act):
    _native.call("b200i_comm_gather_nodes", comm, None, mode, area, ctypes.c_void_p(out.data_ptr()), out.stride(0),
                 ctypes.c_void_p(ws.data_ptr()), nodes, m, n, ctypes.c_void_p(bias.data_ptr()) if bias is not None else None, act)


@pytest.mark.parametrize("kind", ["f32", "int8"])
def test_gather_that_folds_the_leaf_groups(kind):
    """b200i_gemm_w_nodes + b200i_comm_gather_nodes give the words of the finished product followed by the plain
    gather: plain, bias + gelu and gated stores, two ranks emulated on one stream and a world of one."""
    from mojolearn_b200 import torch_ops
    from mojolearn_b200.linalg import OP_NT, W_F32, W_INT8_EXP
    g = torch.Generator(device="cuda").manual_seed(7)
    c0, c1, solo = _create(0, 2, 8 << 20), _create(1, 2, 8 << 20), _create(0, 1, 8 << 20)
    _native.call("b200i_comm_attach_local", c0, 1, c1)
    _native.call("b200i_comm_attach_local", c1, 0, c0)
    split = 0
    cases = ((32, 256, 2048, 0, False), (32, 512, 8192, 0, False), (8, 256, 4096, 1, True), (32, 2048, 2048, 4, False), (5, 64, 6000 - 6000 % 16, 6, True),
             (1, 128, 2048, 0, False))
    for epoch, (m, n, k, act, with_bias) in enumerate(cases):
        for c in (c0, c1, solo):
            _native.call("b200i_comm_advance", c, None)
        if act >= 4 and not _native.lib().b200i_pair_epilogue_fits(m, n, k, OP_NT):
            continue
        x = torch.randn((m, k), generator=g, device="cuda")
        shards = []
        for r in range(2):
            if kind == "int8":
                w = torch.randint(-127, 128, (n, k), generator=g, device="cuda", dtype=torch.int8)
                scale = torch.randint(-12, -4, (n,), generator=g, device="cuda", dtype=torch.int32)
                wk = W_INT8_EXP
            else:
                w, scale, wk = torch.randn((n, k), generator=g, device="cuda"), None, W_F32
            bias = torch.randn((n,), generator=g, device="cuda") if with_bias else None
            shards.append((w, scale, wk, bias))
        want = [torch_ops.product(x, w, s, wk, OP_NT, bias=b, act=act) for (w, s, wk, b) in shards]
        wout = want[0].shape[1]
        parts = [_nodes_product(x, w, s, wk, b, act) for (w, s, wk, b) in shards]
        assert parts[0][2] == parts[1][2]
        if parts[0][2] == 1:  # the plan did not split: the finished product came back
            assert torch.equal(parts[0][0], want[0]) and torch.equal(parts[1][0], want[1]), (m, n, k, act)
            continue
        split += 1
        o0 = torch.full((m, 2 * wout), -1.0, device="cuda")
        o1 = torch.full((m, 2 * wout), -1.0, device="cuda")
        os_ = torch.full((m, wout), -1.0, device="cuda")
        _gather_nodes(c0, SEND, 0, o0, parts[0][1], parts[0][2], m, n, shards[0][3], act)
        _gather_nodes(c1, SEND_RECV, 0, o1, parts[1][1], parts[1][2], m, n, shards[1][3], act)
        _gather(c0, RECV, 0, o0, None)
        _gather_nodes(solo, SEND_RECV, 0, os_, parts[0][1], parts[0][2], m, n, shards[0][3], act)
        torch.cuda.synchronize()
        both = torch.cat(want, dim=1)
        assert torch.equal(o0, both) and torch.equal(o1, both), (m, n, k, act)
        assert torch.equal(os_, want[0]), (m, n, k, act)
    assert split >= 3, split
    assert _native.lib().b200i_decode_status(0) == 0
    for c in (c0, c1, solo):
        _native.lib().b200i_comm_destroy(c)

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

"""The allocation-free product entry point, b200i_gemm_f32_noalloc.

Some callers of this library cannot let it allocate device memory: code that runs
inside an allocator or memory-pool callback, a serving loop that was given a fixed
memory budget up front, or an embedding host that passes raw pointers and forbids
cudaMalloc. For them the split plan's scratch lives in a fixed array inside the
library. This test calls that entry point through the C ABI twice in a row, on
different operands, and holds each result to the ordinary entry point's bits (the
library's parity bar is bit-exact); the second call also shows that the contents the
first call left in the shared scratch do no harm. It also checks the refusal of a shape
whose scratch would not fit. The file name sorts last so that a run that stops at the
first failure has already run every other test.
"""
import ctypes

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native  # noqa: E402


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(a, w, m, n, k, op):
    lib = _native.lib()
    dev = a.device
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    ws_bytes = int(lib.b200i_workspace_bytes(m, n, k))
    want = torch.full((m, n), -987654.0, device=dev)
    ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=dev)
    _native.call("b200i_gemm_f32", dev.index, stream, _vp(want), _vp(a), _vp(w), m, n, k, op, _vp(ws), ws_bytes)
    got = torch.full((m, n), -987654.0, device=dev)
    _native.call("b200i_gemm_f32_noalloc", dev.index, stream, _vp(got), _vp(a), _vp(w), m, n, k, op)
    torch.cuda.synchronize(dev)
    return got, want, ws_bytes


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row():
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(7)
    m, n, k = 320, 192, 4096  # few tiles, 32 leaves: the plan splits the leaves and needs scratch
    used_scratch = False
    for call in range(2):
        a = torch.randn((m, k), generator=g, device=dev)
        w = torch.randn((n, k), generator=g, device=dev)
        got, want, ws_bytes = _both(a, w, m, n, k, 1)
        used_scratch = used_scratch or ws_bytes > 0
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), "call %d" % call
    assert used_scratch, "the chosen shape was meant to exercise the scratch"
    # a second shape, other orientation, odd sizes, right after: stale scratch contents must not matter
    a = torch.randn((1000, 77), generator=g, device=dev)  # op TN: A is [k, m]
    w = torch.randn((1000, 130), generator=g, device=dev)
    got, want, _ = _both(a, w, 77, 130, 1000, 2)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def test_noalloc_refuses_a_shape_beyond_its_scratch():
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    # find a shape whose plan wants more than the 16 MiB built-in scratch
    shape = None
    for m, n, k in ((2048, 2048, 131072), (1536, 1536, 65536), (1024, 4096, 131072)):
        if lib.b200i_workspace_bytes(m, n, k) > (16 << 20):
            shape = (m, n, k)
            break
    if shape is None:
        pytest.skip("no probe shape asks for more than 16 MiB of scratch on this device")
    m, n, k = shape
    a = torch.zeros((4,), device=dev)  # never read: the refusal comes before any launch
    with pytest.raises(_native.NativeError, match="built-in scratch"):
        _native.call("b200i_gemm_f32_noalloc", dev.index, None, _vp(a), _vp(a), _vp(a), m, n, k, 1)

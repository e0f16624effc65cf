"""The allocation-free product entry point, b200i_gemm_f32_noalloc.

Some callers of this library cannot let it allocate device memory: code that runs
inside an allocator or memory-pool callback, a serving loop that was given a fixed
memory budget up front, or an embedding host that passes raw pointers and forbids
cudaMalloc. For them the split plan's scratch lives in a fixed array inside the
library. This test calls that entry point through the C ABI twice in a row, on
different operands, and holds each result to the ordinary entry point's bits (the
library's parity bar is bit-exact); the second call also shows that the contents the
first call left in the shared scratch do no harm. It checks that a warmed-up call
leaves the device's free memory untouched, and that a shape whose preferred leaf
split would not fit the built-in scratch is still computed, bit for bit, with a
coarser split. The file name sorts last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native  # noqa: E402

SCRATCH = 16 << 20


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(a, w, m, n, k, op):
    lib = _native.lib()
    dev = a.device
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    ws_bytes = int(lib.b200i_workspace_bytes(m, n, k))
    want = torch.full((m, n), -987654.0, device=dev)
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device=dev)
    _native.call("b200i_gemm_f32", dev.index, stream, _vp(want), _vp(a), _vp(w), m, n, k, op, _vp(ws), ws_bytes)
    got = torch.full((m, n), -987654.0, device=dev)
    _native.call("b200i_gemm_f32_noalloc", dev.index, stream, _vp(got), _vp(a), _vp(w), m, n, k, op)
    torch.cuda.synchronize(dev)
    return got, want


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row():
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(7)
    m, n, k = 320, 192, 4096  # few tiles, 32 leaves: the plan splits the leaves and needs scratch
    assert 0 < _native.lib().b200i_noalloc_scratch_bytes(m, n, k) <= SCRATCH, "the chosen shape was meant to exercise the scratch"
    for call in range(2):
        a = torch.randn((m, k), generator=g, device=dev)
        w = torch.randn((n, k), generator=g, device=dev)
        got, want = _both(a, w, m, n, k, 1)
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), "call %d" % call
    # a second shape, other orientation, odd sizes, right after: stale scratch contents must not matter
    a = torch.randn((1000, 77), generator=g, device=dev)  # op TN: A is [k, m]
    w = torch.randn((1000, 130), generator=g, device=dev)
    got, want = _both(a, w, 77, 130, 1000, 2)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def test_noalloc_leaves_free_memory_untouched_once_warm():
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(8)
    m, n, k = 320, 192, 4096
    a = torch.randn((m, k), generator=g, device=dev)
    w = torch.randn((n, k), generator=g, device=dev)
    c = torch.empty((m, n), device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    _native.call("b200i_gemm_f32_noalloc", dev.index, stream, _vp(c), _vp(a), _vp(w), m, n, k, 1)  # warm: kernels loaded, address known
    torch.cuda.synchronize(dev)
    free0, _ = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        _native.call("b200i_gemm_f32_noalloc", dev.index, stream, _vp(c), _vp(a), _vp(w), m, n, k, 1)
    torch.cuda.synchronize(dev)
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0, "a warmed-up allocation-free call changed the device's free memory"


def test_noalloc_runs_a_coarser_split_when_the_preferred_one_does_not_fit():
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    m, n, k = 128, 11008, 4096  # the ordinary entry's preferred split wants far more than 16 MiB of group nodes here
    assert lib.b200i_noalloc_scratch_bytes(m, n, k) <= SCRATCH
    g = torch.Generator(device=dev).manual_seed(9)
    a = torch.randn((m, k), generator=g, device=dev)
    w = torch.randn((n, k), generator=g, device=dev)
    got, want = _both(a, w, m, n, k, 1)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    # no shape is refused for its scratch: even a deep product with few tiles reports a need within the array
    for shape in ((2048, 2048, 131072), (1536, 1536, 65536), (1024, 4096, 131072), (4096, 4096, 4096), (2048, 50304, 768)):
        assert 0 <= lib.b200i_noalloc_scratch_bytes(*shape) <= SCRATCH, shape
    # the ordinary refusals still come before any launch: null storage is named, nothing is read or written
    with pytest.raises(_native.NativeError, match="null storage"):
        _native.call("b200i_gemm_f32_noalloc", dev.index, None, None, None, None, m, n, k, 1)

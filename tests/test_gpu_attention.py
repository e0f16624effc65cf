"""The attention entry points against the CPU oracle at serving sizes.

`b200i_attention` and `b200i_attention_at` (the position read from a device word, as a replayed CUDA graph needs it)
with 1, 2, 4 and 8 query rows per sequence -- the decode-step kernels -- at head_dim 128 and 64, on caches of
31 ... 1279 positions: around the edges of a 32-key tile, past the point where the value ring refills a slot (more
than 96 keys), and at the serving benchmark's lengths; with and without a sliding window, with grouped-query heads,
and with operands that make a late tile fail the admission test of the bare multiply-add, so that the flushed chain
has to take over in the middle of a row. Bit for bit, against oracle/decoder_oracle.c's dec_attention, which follows
transformer/checks/transformer_oracle.mojo:2373-2546 of the reference (S11-S19).
"""
import ctypes

import numpy as np
import pytest

import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native  # noqa: E402

KEYS = (31, 32, 33, 95, 96, 97, 129, 1030, 1279)


def _vp(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _run(q, kc, vc, l, used, window, at, softcap=0.0):
    """ctx through the C ABI; `at` = the device-position twin."""
    b, nkv, cap, hd = kc.shape
    nh = q.shape[1]
    dq, dk, dv = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (q, kc, vc))
    ctx = torch.full((b * l, nh * hd), np.float32(-777.0), device="cuda")
    if at:
        smax = min(cap, window - 1 + l) if window else cap
        scores = torch.empty((b * nh * l * smax,), device="cuda")
        pos = torch.tensor([used - l], dtype=torch.int32, device="cuda")
        _native.call("b200i_attention_at", 0, None, _vp(ctx), _vp(dq), _vp(dk), _vp(dv), _vp(scores), b, l, nh, nkv, hd, cap,
                     _vp(pos), window, softcap)
    else:
        s = used - (max(0, used - l - (window - 1)) if window else 0)
        scores = torch.empty((b * nh * l * s,), device="cuda")
        _native.call("b200i_attention", 0, None, _vp(ctx), _vp(dq), _vp(dk), _vp(dv), _vp(scores), b, l, nh, nkv, hd, cap, used,
                     window, softcap)
    torch.cuda.synchronize()
    assert _native.lib().b200i_decode_status(0) == 0
    return ctx.cpu().numpy()


def _operands(rng, b, l, nh, nkv, hd, cap, scale_q=1.0):
    q = (rng.standard_normal((b * l, nh, hd)) * scale_q).astype(np.float32)
    kc = rng.standard_normal((b, nkv, cap, hd)).astype(np.float32)
    vc = rng.standard_normal((b, nkv, cap, hd)).astype(np.float32)
    return q, kc, vc


@pytest.mark.parametrize("hd", (128, 64))
@pytest.mark.parametrize("l", (1, 2, 4, 8))
def test_decode_step_attention_at_tile_edges_and_serving_lengths(l, hd):
    rng = np.random.default_rng(1000 * l + hd)
    b, nh, nkv, cap = 2, 4, 4, 1280
    q, kc, vc = _operands(rng, b, l, nh, nkv, hd, cap, 0.3)
    for used in KEYS:
        if used < l:
            continue
        want = oracle.attention(q, kc, vc, l, used)
        for at in (False, True):
            got = _run(q, kc, vc, l, used, 0, at)
            assert got.tobytes() == want.tobytes(), (l, hd, used, at)


@pytest.mark.parametrize("hd", (128, 64))
def test_decode_step_attention_window_and_grouped_heads(hd):
    rng = np.random.default_rng(7 + hd)
    b, nh, nkv, cap = 3, 6, 2, 1100
    for l in (1, 4):
        q, kc, vc = _operands(rng, b, l, nh, nkv, hd, cap, 0.3)
        for used, window in ((33, 0), (97, 40), (129, 100), (1030, 0), (1030, 333), (1030, 31), (1099, 64)):
            want = oracle.attention(q, kc, vc, l, used, window)
            for at in (False, True):
                got = _run(q, kc, vc, l, used, window, at)
                assert got.tobytes() == want.tobytes(), (l, hd, used, window, at)


@pytest.mark.parametrize("l", (1, 8))
def test_decode_step_attention_admission_fails_in_a_late_tile(l):
    """Subnormal-forcing operands in the last tiles only: tiny values (the value chain's products fall below 2^-126)
    and tiny keys (the score chain's), after hundreds of ordinary keys; and one subnormal word in the middle."""
    rng = np.random.default_rng(99 + l)
    b, nh, nkv, hd, cap, used = 2, 2, 1, 128, 1100, 1030
    q, kc, vc = _operands(rng, b, l, nh, nkv, hd, cap, 0.3)
    tiny = np.float32(2.0 ** -100)
    for variant in range(4):
        k2, v2, q2 = kc.copy(), vc.copy(), q.copy()
        if variant == 0:
            v2[:, :, 990:, :] *= tiny
        elif variant == 1:
            k2[:, :, 1000:, :] *= tiny
            q2 *= np.float32(2.0 ** -40)
        elif variant == 2:
            v2[0, 0, 517, 5] = np.float32(1e-41)
            k2[1, 0, 700, 77] = np.float32(-1e-42)
        else:
            v2[:, :, 64:96, :] *= np.float32(2.0 ** -120)  # a whole middle tile, ordinary tiles on both sides
        want = oracle.attention(q2, k2, v2, l, used)
        for at in (False, True):
            got = _run(q2, k2, v2, l, used, 0, at)
            assert got.tobytes() == want.tobytes(), (l, variant, at)


def test_prefill_attention_against_the_oracle_at_head_dim_128_and_64():
    """A prompt-sized call (l > 8 takes the tiled kernels): 200 and 77 positions on an empty and on a part-filled cache."""
    rng = np.random.default_rng(5)
    for hd, l, used, window in ((128, 200, 200, 0), (64, 77, 300, 0), (128, 130, 130, 50), (64, 33, 1030, 0)):
        b, nh, nkv, cap = 2, 4, 2, max(used, 64)
        q, kc, vc = _operands(rng, b, l, nh, nkv, hd, cap, 0.3)
        want = oracle.attention(q, kc, vc, l, used, window)
        got = _run(q, kc, vc, l, used, window, False)
        assert got.tobytes() == want.tobytes(), (hd, l, used, window)

"""GPU parity for the weight-storage paths: conversions, the int8 / bf16 weight
products at decode and prefill row counts (the serving benchmark's Llama-7B projection shapes), and the
launch invariance of the decode plan against the tiled and flat plans."""
import numpy as np
import pytest

import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native, linalg, lowbit, torch_ops  # noqa: E402


def test_conversions_match_the_oracle():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((257, 131)) * np.exp2(rng.integers(-140, 120, (257, 1)))).astype(np.float32)
    x[0, :5] = [np.nan, np.inf, -np.inf, 1e-41, -1e-41]
    assert linalg.to_bf16(x).tobytes() == oracle.to_bf16(x).tobytes()
    bits = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    assert linalg.from_bf16(bits).tobytes() == oracle.from_bf16(bits).tobytes()
    allf = oracle.from_bf16(bits)
    assert linalg.to_bf16(allf).tobytes() == oracle.to_bf16(allf).tobytes()
    q, e = linalg.quantize_int8(x)
    qo, eo = oracle.quantize_int8(x)
    assert q.tobytes() == qo.tobytes() and e.tobytes() == eo.tobytes()
    assert linalg.dequantize_int8(q, e).tobytes() == oracle.dequantize_int8(qo, eo).tobytes()
    x3 = rng.standard_normal((5, 7, 9)).astype(np.float32)
    assert linalg.to_bf16(x3).shape == (5, 7, 9)
    odd = rng.standard_normal(1001).astype(np.float32)[1:]  # misaligned, odd count
    assert linalg.to_bf16(odd).tobytes() == oracle.to_bf16(odd).tobytes()


def test_lowbit_pack_roundtrip():
    rng = np.random.default_rng(1)
    w = {"q": (rng.standard_normal((64, 48)) * 0.02).astype(np.float32), "norm": np.ones(48, np.float32)}
    for fmt in ("bfloat16", "int8", "float32"):
        packed = lowbit.pack(w, fmt)
        assert lowbit.format_of(packed) == fmt and packed["norm"] is w["norm"]
        mat = lowbit.unpack(packed)
        if fmt == "int8":
            q, e = oracle.quantize_int8(w["q"])
            assert mat["q"].tobytes() == oracle.dequantize_int8(q, e).tobytes()
        elif fmt == "bfloat16":
            assert mat["q"].tobytes() == oracle.from_bf16(oracle.to_bf16(w["q"])).tobytes()


def _weights(n, k, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
    scales = rng.uniform(0.001, 0.02, n).astype(np.float32)
    exps = np.round(np.log2(scales)).astype(np.int32)  # snapped to powers of two: the reference's format
    wb = oracle.to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    return codes, scales, exps, wb


@pytest.mark.parametrize("m", [1, 2, 5, 8, 32, 128])
def test_config3_reduced_n_against_the_scalar_oracle(m):
    n, k = 520, 4096
    codes, scales, exps, wb = _weights(n, k, 3)
    x = np.random.default_rng(4).standard_normal((m, k)).astype(np.float32)
    w8 = oracle.dequantize_int8(codes, exps)
    assert linalg.matmul_int8w(x, codes, exps).tobytes() == oracle.gemm(x, w8, oracle.OP_NT).tobytes()
    w8s = oracle.dequantize_int8_scaled(codes, scales)  # extension: general float32 scales (parity unpinned)
    assert linalg.matmul_int8w(x, codes, scales=scales).tobytes() == oracle.gemm(x, w8s, oracle.OP_NT).tobytes()
    wf = oracle.from_bf16(wb)
    assert linalg.matmul_bf16(x, wb, transpose_b=True).tobytes() == oracle.gemm(x, wf, oracle.OP_NT).tobytes()
    assert linalg.matmul(x, wf, transpose_b=True).tobytes() == oracle.gemm(x, wf, oracle.OP_NT).tobytes()


@pytest.mark.parametrize("m", [1, 8, 32, 128])
def test_config3_full_size(m):
    """W [11008, 4096]: the whole product on the GPU against the threaded CPU
    oracle (m <= 8), or sampled columns of it (larger m), plus plan invariance."""
    n, k = 11008, 4096
    codes, scales, exps, wb = _weights(n, k, 5)
    x = np.random.default_rng(6).standard_normal((m, k)).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    dcodes, dexps, dscales, dwb = (torch.from_numpy(v).cuda() for v in (codes, exps, scales, wb))
    got8 = torch_ops.linear_int8w(dx, dcodes, exponents=dexps)
    gots = torch_ops.linear_int8w(dx, dcodes, scales=dscales)
    gotb = torch_ops.matmul_bf16(dx, dwb, transpose_b=True)
    cols = np.arange(n) if m <= 8 else np.sort(np.random.default_rng(7).choice(n, 600, replace=False))
    w8 = oracle.dequantize_int8(codes[cols], exps[cols])
    assert got8.cpu().numpy()[:, cols].tobytes() == oracle.gemm_rows(x, w8, oracle.OP_NT).tobytes()
    w8s = oracle.dequantize_int8_scaled(codes[cols], scales[cols])
    assert gots.cpu().numpy()[:, cols].tobytes() == oracle.gemm_rows(x, w8s, oracle.OP_NT).tobytes()
    wf = oracle.from_bf16(wb[cols])
    assert gotb.cpu().numpy()[:, cols].tobytes() == oracle.gemm_rows(x, wf, oracle.OP_NT).tobytes()
    # every plan that accepts the shape returns the same words
    fits = _native.lib().b200i_decode_plan_fits(m, n, k, oracle.OP_NT, linalg.W_INT8_EXP)
    assert fits == (1 if m <= 8 else 0)
    plans = [(torch_ops.PLAN_T128, 0), (torch_ops.PLAN_T64, 4), (torch_ops.PLAN_PACKED, 0), (torch_ops.PLAN_PACKED, 4)]
    plans += [(torch_ops.PLAN_DECODE, 0)] if fits else []
    plans += [(torch_ops.PLAN_SKINNY, 0), (torch_ops.PLAN_SKINNY, 2)] if m <= 32 else []
    for plan, groups in plans:
        alt = torch_ops.product(dx, dcodes, dexps, linalg.W_INT8_EXP, oracle.OP_NT, plan=plan, group_leaves=groups)
        assert torch.equal(alt.view(torch.int32), got8.view(torch.int32)), (plan, groups)
        altb = torch_ops.product(dx, dwb, None, linalg.W_BF16, oracle.OP_NT, plan=plan, group_leaves=groups)
        assert torch.equal(altb.view(torch.int32), gotb.view(torch.int32)), (plan, groups)
    assert _native.lib().b200i_decode_status(-1) == 0


def test_decode_plan_edges():
    """Ragged row counts per CTA, k below one leaf, k with a short last leaf,
    subnormal-forcing weights and activations, exotic exponents."""
    rng = np.random.default_rng(8)
    for (m, n, k) in [(1, 7, 16), (3, 33, 128), (8, 1000, 1040), (2, 4097, 2048), (4, 300, 8192), (8, 70, 8192), (1, 50304, 768), (8, 48, 384)]:
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        dx, dw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        want = oracle.gemm_rows(x, w, oracle.OP_NT)
        got = torch_ops.product(dx, dw, None, linalg.W_F32, oracle.OP_NT, plan=torch_ops.PLAN_DECODE)
        assert got.cpu().numpy().tobytes() == want.tobytes(), (m, n, k)
        assert _native.lib().b200i_decode_status(-1) == 0, (m, n, k)
    m, n, k = 4, 200, 512
    x = (rng.standard_normal((m, k)) * 2.0 ** -62).astype(np.float32)
    x[0, ::9] = np.float32(3e-42)
    codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
    exps = rng.integers(-70, -58, n).astype(np.int32)
    exps[:4] = [-140, 127, 121, -127]
    w = oracle.dequantize_int8(codes, exps)
    want = oracle.nan_canon(oracle.gemm(x, w, oracle.OP_NT))
    dx, dc, de = torch.from_numpy(x).cuda(), torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda()
    for plan in (torch_ops.PLAN_DECODE, torch_ops.PLAN_T64, torch_ops.PLAN_FLAT, torch_ops.PLAN_AUTO, torch_ops.PLAN_PACKED):
        got = torch_ops.product(dx, dc, de, linalg.W_INT8_EXP, oracle.OP_NT, plan=plan)
        assert got.cpu().numpy().tobytes() == want.tobytes(), plan
    scales = (rng.uniform(0.5, 2.0, n) * 2.0 ** -66).astype(np.float32)
    scales[:4] = [np.float32(2e-42), np.float32(3e37), np.float32(1.0), np.float32(0.0)]
    wants = oracle.nan_canon(oracle.gemm(x, oracle.dequantize_int8_scaled(codes, scales), oracle.OP_NT))
    got = torch_ops.product(dx, torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda(), linalg.W_INT8_SCALE, oracle.OP_NT,
                            plan=torch_ops.PLAN_SKINNY)
    assert got.cpu().numpy().tobytes() == wants.tobytes()
    wb = oracle.to_bf16((rng.standard_normal((n, k)) * 2.0 ** -64).astype(np.float32))
    wantb = oracle.gemm(x, oracle.from_bf16(wb), oracle.OP_NT)
    for plan in (torch_ops.PLAN_DECODE, torch_ops.PLAN_T128, torch_ops.PLAN_PACKED):
        got = torch_ops.product(dx, torch.from_numpy(wb).cuda(), None, linalg.W_BF16, oracle.OP_NT, plan=plan)
        assert got.cpu().numpy().tobytes() == wantb.tobytes(), plan
    assert _native.lib().b200i_decode_status(-1) == 0


def test_skinny_plan_every_storage_kind():
    """The skinny plan (up to 32 activation rows): ragged row and column counts,
    one to many leaves per group, a short last leaf, every storage kind, and
    operands that force the flushed path."""
    rng = np.random.default_rng(11)
    shapes = [(5, 300, 512, 0), (8, 1030, 4096, 8), (9, 520, 2048, 4), (16, 1000, 1024, 0), (17, 700, 4096, 16),
              (32, 513, 2048, 2), (32, 256, 64, 0), (12, 99, 4096 + 128, 8), (3, 2050, 768, 2), (1, 40, 16, 0),
              (8, 260, 8192, 1), (5, 99, 128 * 43, 1),  # 64 and 43 leaf groups: the group fold's full and ragged stacks
              (32, 768, 2048, 1), (27, 600, 2048, 1)]  # 48 CTAs of 32 rows: the low-bit kernel splits the rows once (16 + 16, 16 + 11)
    for (m, n, k, gl) in shapes:
        x = rng.standard_normal((m, k)).astype(np.float32)
        codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
        exps = rng.integers(-9, -5, n).astype(np.int32)
        scales = rng.uniform(0.001, 0.02, n).astype(np.float32)
        wb = oracle.to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        wf = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        dx = torch.from_numpy(x).cuda()
        cases = [(wf, None, linalg.W_F32, wf), (wb, None, linalg.W_BF16, oracle.from_bf16(wb)),
                 (codes, exps, linalg.W_INT8_EXP, oracle.dequantize_int8(codes, exps)),
                 (codes, scales, linalg.W_INT8_SCALE, oracle.dequantize_int8_scaled(codes, scales))]
        for w, sc, kind, wref in cases:
            want = oracle.gemm_rows(x, wref, oracle.OP_NT)
            got = torch_ops.product(dx, torch.from_numpy(w).cuda(), None if sc is None else torch.from_numpy(sc).cuda(), kind,
                                    oracle.OP_NT, plan=torch_ops.PLAN_SKINNY, group_leaves=gl)
            assert got.cpu().numpy().tobytes() == want.tobytes(), (m, n, k, gl, kind)
    m, n, k = 12, 200, 512
    x = (rng.standard_normal((m, k)) * 2.0 ** -62).astype(np.float32)
    x[0, ::9] = np.float32(3e-42)
    codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
    exps = rng.integers(-70, -58, n).astype(np.int32)
    exps[:4] = [-140, 127, 121, -127]
    want = oracle.nan_canon(oracle.gemm(x, oracle.dequantize_int8(codes, exps), oracle.OP_NT))
    dx = torch.from_numpy(x).cuda()
    for plan in (torch_ops.PLAN_SKINNY, torch_ops.PLAN_AUTO):
        got = torch_ops.product(dx, torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda(), linalg.W_INT8_EXP, oracle.OP_NT, plan=plan)
        assert got.cpu().numpy().tobytes() == want.tobytes(), plan
    scales = (rng.uniform(0.5, 2.0, n) * 2.0 ** -66).astype(np.float32)
    scales[:4] = [np.float32(2e-42), np.float32(3e37), np.float32(1.0), np.float32(0.0)]
    wants = oracle.nan_canon(oracle.gemm(x, oracle.dequantize_int8_scaled(codes, scales), oracle.OP_NT))
    got = torch_ops.product(dx, torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda(), linalg.W_INT8_SCALE, oracle.OP_NT,
                            plan=torch_ops.PLAN_SKINNY)
    assert got.cpu().numpy().tobytes() == wants.tobytes()
    wb = oracle.to_bf16((rng.standard_normal((n, k)) * 2.0 ** -64).astype(np.float32))
    wantb = oracle.gemm(x, oracle.from_bf16(wb), oracle.OP_NT)
    got = torch_ops.product(dx, torch.from_numpy(wb).cuda(), None, linalg.W_BF16, oracle.OP_NT, plan=torch_ops.PLAN_SKINNY)
    assert got.cpu().numpy().tobytes() == wantb.tobytes()
    # refusals: more than 32 rows, k not a multiple of 16, another op
    with pytest.raises(_native.NativeError):
        torch_ops.product(torch.zeros(33, 64).cuda(), torch.zeros(8, 64).cuda(), None, linalg.W_F32, oracle.OP_NT, plan=torch_ops.PLAN_SKINNY)
    with pytest.raises(_native.NativeError):
        torch_ops.product(torch.zeros(4, 40).cuda(), torch.zeros(8, 40).cuda(), None, linalg.W_F32, oracle.OP_NT, plan=torch_ops.PLAN_SKINNY)
    with pytest.raises(_native.NativeError):
        torch_ops.product(torch.zeros(4, 64).cuda(), torch.zeros(64, 8).cuda(), None, linalg.W_F32, oracle.OP_NN, plan=torch_ops.PLAN_SKINNY)


def test_int8_product_profile():
    rng = np.random.default_rng(9)
    a = rng.standard_normal((37, 1000)).astype(np.float32)
    b = rng.standard_normal((41, 1000)).astype(np.float32)
    qa, ea = oracle.quantize_int8(a)
    qb, eb = oracle.quantize_int8(b)
    assert linalg.matmul_int8((qa, ea), (qb, eb)).tobytes() == oracle.gemm_int8(qa, ea, qb, eb).tobytes()
    assert linalg.matmul_int8(a, b).tobytes() == oracle.gemm_int8(qa, ea, qb, eb).tobytes()


def test_int8_product_on_tensor_cores():
    """k a multiple of 16: the product runs as tcgen05 int8 MMAs into an int32 accumulator in tensor memory. Ragged tiles
    in m and n, k below / at / across the 128-byte stage, the largest sums an int32 can hold, extreme exponents."""
    rng = np.random.default_rng(10)
    for (m, n, k) in [(1, 7, 16), (37, 41, 1008), (128, 128, 128), (130, 257, 400), (300, 515, 4096), (5, 129, 144), (2048, 2600, 272), (1300, 4100, 640), (256, 70003, 64)]:
        qa = rng.integers(-127, 128, (m, k)).astype(np.int8)
        qb = rng.integers(-127, 128, (n, k)).astype(np.int8)
        ea = rng.integers(-20, 20, m).astype(np.int32)
        eb = rng.integers(-20, 20, n).astype(np.int32)
        assert linalg.matmul_int8((qa, ea), (qb, eb)).tobytes() == oracle.gemm_int8(qa, ea, qb, eb).tobytes(), (m, n, k)
    m, n, k = 3, 5, 131072  # |sum| up to 127 * 127 * 131072 < 2^31
    qa = np.full((m, k), 127, np.int8)
    qb = np.full((n, k), 127, np.int8)
    qa[1] = -127
    qb[2, ::2] = -128
    qa[2, : k // 2] = 0
    ea = np.array([0, -140, 100], np.int32)
    eb = np.array([0, 120, -130, 5, -5], np.int32)
    assert linalg.matmul_int8((qa, ea), (qb, eb)).tobytes() == oracle.gemm_int8(qa, ea, qb, eb).tobytes()
    assert _native.lib().b200i_decode_status(-1) == 0


def test_int15_profile_against_the_oracle():
    """The fifteen-bit profile: quantiser (planes and exponents, NaN / Inf / zero / tiny rows), dequantiser, and the product on
    the tensor cores (k a multiple of 16: ragged tiles, k below / at / across a stage, the largest codes at the largest k)
    and one thread per cell (any other k), against the CPU oracle, which reproduces the reference's `gemm-int15` cells."""
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((67, 131)) * np.exp2(rng.integers(-140, 120, (67, 1)))).astype(np.float32)
    x[0, :6] = [np.nan, np.inf, -np.inf, 1e-41, -1e-41, 0.0]
    x[1] = 0.0
    x[2, :] = np.float32(1e-40)
    x[3, 5] = np.nan
    hi, lo, e = linalg.quantize_int15(x)
    ohi, olo, oe = oracle.quantize_int15(x)
    assert hi.tobytes() == ohi.tobytes() and lo.tobytes() == olo.tobytes() and e.tobytes() == oe.tobytes()
    assert linalg.dequantize_int15(hi, lo, e).tobytes() == oracle.dequantize_int15(ohi, olo, oe).tobytes()
    for (m, n, k) in [(1, 7, 16), (37, 41, 1008), (128, 64, 128), (130, 257, 400), (300, 515, 2048), (5, 129, 144), (1300, 2100, 640),
                      (37, 41, 1000), (3, 5, 7), (130, 70003, 48)]:
        a = (rng.standard_normal((m, k)) * np.exp2(rng.integers(-20, 20, (m, 1)))).astype(np.float32)
        b = (rng.standard_normal((n, k)) * np.exp2(rng.integers(-20, 20, (n, 1)))).astype(np.float32)
        qa, qb = oracle.quantize_int15(a), oracle.quantize_int15(b)
        want = oracle.nan_canon(oracle.gemm_int15(*qa, *qb))
        assert linalg.matmul_int15(qa, qb).tobytes() == want.tobytes(), (m, n, k)
        assert linalg.matmul_int15(a, b).tobytes() == want.tobytes(), (m, n, k)
    m, n, k = 3, 5, 65536  # |sum| up to 16383^2 * 65536 < 2^44: every piece sum at its bound
    ah = np.full((m, k), 127, np.int8); al = np.full((m, k), 127, np.int8)
    bh = np.full((n, k), 127, np.int8); bl = np.full((n, k), 127, np.int8)
    ah[1] = -128; al[1] = 1
    bh[2, ::2] = -128; bl[2, ::2] = 1
    al[2, : k // 2] = 0
    ea = np.array([0, -140, 100], np.int32)
    eb = np.array([0, 120, -130, 5, -5], np.int32)
    want = oracle.nan_canon(oracle.gemm_int15(ah, al, ea, bh, bl, eb))
    assert linalg.matmul_int15((ah, al, ea), (bh, bl, eb)).tobytes() == want.tobytes()
    with pytest.raises(ValueError, match="65536"):
        linalg.matmul_int15(np.zeros((1, 65537), np.float32), np.zeros((1, 65537), np.float32))
    assert _native.lib().b200i_decode_status(-1) == 0


@pytest.mark.parametrize("chunk", range(4))
def test_skinny_register_plan_over_leaf_counts(chunk):
    """The register skinny plan (low-bit weights) over every leaf count from 1 to 40 and a few up to 1024, leaf groups
    of 1, 2, 4 and 8 (ragged last groups included), 8, 16 and 32-row tiles, int8 and bf16 weights, two column tiles
    with a ragged edge: the bits of the oracle's tree."""
    counts = (list(range(1, 41)) + [48, 63, 64, 65, 100, 255, 256, 257, 1000, 1024])[chunk::4]
    n = 300
    for p in counts:
        k = (p - 1) * 128 + (128 if p % 2 == 0 else 32)
        rng = np.random.default_rng(1000 + p)
        m = (3, 8, 13, 32)[p % 4]
        x = (rng.standard_normal((m, k)) * np.exp2(rng.integers(-10, 11, (m, k)))).astype(np.float32)
        w = (rng.standard_normal((n, k)) * np.exp2(rng.integers(-10, 11, (n, k)))).astype(np.float32)
        dx = torch.from_numpy(x).cuda()
        codes, exps = oracle.quantize_int8(w)
        bits = oracle.to_bf16(w)
        for kind, dw, ds, wf in ((linalg.W_INT8_EXP, torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda(), oracle.dequantize_int8(codes, exps)),
                                 (linalg.W_BF16, torch.from_numpy(bits).cuda(), None, oracle.from_bf16(bits))):
            if kind == linalg.W_BF16 and p > 40:
                continue
            want = oracle.nan_canon(oracle.gemm_rows(x, wf, oracle.OP_NT))
            for plan in (torch_ops.PLAN_SKINNY, torch_ops.PLAN_AUTO):
                for gl in ((0,) if plan == torch_ops.PLAN_AUTO else (0, 1, 2, 4, 8)):
                    if gl and (p + gl - 1) // gl > 64:
                        continue
                    got = torch_ops.product(dx, dw, ds, kind, oracle.OP_NT, plan=plan, group_leaves=gl)
                    assert got.cpu().numpy().tobytes() == want.tobytes(), (p, m, kind, plan, gl)
    assert _native.lib().b200i_decode_status(-1) == 0


@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_leaf_pair_decode_kernel(m):
    """Weights wide enough (n >= 16 rows per SM) that the decode plan takes its leaf-pair kernel for bf16 / int8 at one to
    four activation rows: k below one leaf, short last leaves, leaf counts that leave the lane fold an odd tail, a row count
    that leaves the last block of a CTA ragged; then operands that fail admission (the flushed per-row fallback) and row
    scales outside the range of the one-fma dequantisation."""
    rng = np.random.default_rng(20 + m)
    n = 2403 + 8 * 148  # > 16 * 148 rows, odd
    dec = torch_ops.PLAN_DECODE
    for k in (16, 112, 128, 144, 400, 1024, 1168, 2048, 2112, 4096, 11008):
        codes, scales, exps, wb = _weights(n, k, 30 + k)
        x = rng.standard_normal((m, k)).astype(np.float32)
        dx = torch.from_numpy(x).cuda()
        got = torch_ops.product(dx, torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda(), linalg.W_INT8_EXP, oracle.OP_NT, plan=dec)
        assert got.cpu().numpy().tobytes() == oracle.gemm_rows(x, oracle.dequantize_int8(codes, exps), oracle.OP_NT).tobytes(), ("int8", k)
        got = torch_ops.product(dx, torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda(), linalg.W_INT8_SCALE, oracle.OP_NT, plan=dec)
        assert got.cpu().numpy().tobytes() == oracle.gemm_rows(x, oracle.dequantize_int8_scaled(codes, scales), oracle.OP_NT).tobytes(), ("int8s", k)
        got = torch_ops.product(dx, torch.from_numpy(wb).cuda(), None, linalg.W_BF16, oracle.OP_NT, plan=dec)
        assert got.cpu().numpy().tobytes() == oracle.gemm_rows(x, oracle.from_bf16(wb), oracle.OP_NT).tobytes(), ("bf16", k)
        assert _native.lib().b200i_decode_status(-1) == 0, k
    # admission fails: tiny activations with subnormals among them, small weights; exotic exponents and scales on some rows
    k = 1168
    x = (rng.standard_normal((m, k)) * 2.0 ** -62).astype(np.float32)
    x[0, ::9] = np.float32(3e-42)
    codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
    exps = rng.integers(-70, -58, n).astype(np.int32)
    exps[:6] = [-140, 127, 121, -127, -101, 101]
    exps[1000:1003] = [-150, 100, -126]
    dx, dc = torch.from_numpy(x).cuda(), torch.from_numpy(codes).cuda()
    want = oracle.nan_canon(oracle.gemm_rows(x, oracle.dequantize_int8(codes, exps), oracle.OP_NT))
    got = torch_ops.product(dx, dc, torch.from_numpy(exps).cuda(), linalg.W_INT8_EXP, oracle.OP_NT, plan=dec)
    assert got.cpu().numpy().tobytes() == want.tobytes()
    scales = (rng.uniform(0.5, 2.0, n) * 2.0 ** -66).astype(np.float32)
    scales[:5] = [np.float32(2e-42), np.float32(3e37), np.float32(1.0), np.float32(0.0), np.float32(-0.75)]
    want = oracle.nan_canon(oracle.gemm_rows(x, oracle.dequantize_int8_scaled(codes, scales), oracle.OP_NT))
    got = torch_ops.product(dx, dc, torch.from_numpy(scales).cuda(), linalg.W_INT8_SCALE, oracle.OP_NT, plan=dec)
    assert got.cpu().numpy().tobytes() == want.tobytes()
    wb = oracle.to_bf16((rng.standard_normal((n, k)) * 2.0 ** -64).astype(np.float32))
    want = oracle.nan_canon(oracle.gemm_rows(x, oracle.from_bf16(wb), oracle.OP_NT))
    got = torch_ops.product(dx, torch.from_numpy(wb).cuda(), None, linalg.W_BF16, oracle.OP_NT, plan=dec)
    assert got.cpu().numpy().tobytes() == want.tobytes()
    # ordinary activations against weights of which only a few rows fail admission
    x = rng.standard_normal((m, k)).astype(np.float32)
    wf = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    wf[5] *= np.float32(2.0 ** -120)
    wf[n - 2, 100:130] = np.float32(1e-40)
    wb = oracle.to_bf16(wf)
    want = oracle.nan_canon(oracle.gemm_rows(x, oracle.from_bf16(wb), oracle.OP_NT))
    got = torch_ops.product(torch.from_numpy(x).cuda(), torch.from_numpy(wb).cuda(), None, linalg.W_BF16, oracle.OP_NT, plan=dec)
    assert got.cpu().numpy().tobytes() == want.tobytes()
    assert _native.lib().b200i_decode_status(-1) == 0

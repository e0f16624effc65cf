"""GPU parity for the fp32 product: the CUDA path, through the C ABI, against the
CPU oracle, bit for bit. Modelled on the reference's device gates
(gemm/checks/gemm_device_check.mojo: device == oracle :840, launch invariance
:1016, batch invariance :1464) and its Python-surface gate
(python/mojolearn/tests/test_linalg_identity.py: shapes chosen by leaf count
with m, n, k pairwise distinct, :382-412)."""
import ctypes

import numpy as np
import pytest

import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native, linalg, torch_ops  # noqa: E402

OPS = {"NN": oracle.OP_NN, "NT": oracle.OP_NT, "TN": oracle.OP_TN}
PLANS = [(torch_ops.PLAN_FLAT, 0), (torch_ops.PLAN_T128, 0), (torch_ops.PLAN_T64, 0), (torch_ops.PLAN_T128, 1),
         (torch_ops.PLAN_T64, 2), (torch_ops.PLAN_T128, 4), (torch_ops.PLAN_T32, 0), (torch_ops.PLAN_T32, 2),
         (torch_ops.PLAN_PACKED, 0), (torch_ops.PLAN_PACKED, 2)]

# (m, n, k): P = 1, 2, 3 (ragged, odd carry), 5 (carries twice), 6, 8 with a short last leaf, tails, k = 1
SHAPES = [(40, 20, 300), (11, 6, 640), (9, 5, 256), (17, 3, 64), (8, 48, 384), (36, 9, 300), (1, 1, 1), (5, 7, 1),
          (130, 70, 129), (257, 131, 768), (100, 100, 1000), (64, 192, 128), (3, 515, 136), (129, 257, 2049)]


def _operands(m, n, k, op, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((k, m) if op == oracle.OP_TN else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if op == oracle.OP_NT else (k, n)).astype(np.float32)
    return a, b


def _gpu(a, b, op, plan=torch_ops.PLAN_AUTO, groups=0):
    c = torch_ops.product(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), None, linalg.W_F32, op, plan=plan,
                          group_leaves=groups)
    return c.cpu().numpy()


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("opname", ["NN", "NT", "TN"])
def test_device_matches_oracle_on_every_plan(m, n, k, opname):
    op = OPS[opname]
    a, b = _operands(m, n, k, op, m * 7 + n * 3 + k)
    want = oracle.nan_canon(oracle.gemm(a, b, op))
    assert _gpu(a, b, op).tobytes() == want.tobytes()
    leaves = oracle.leaf_count(k)
    for plan, groups in PLANS:
        if groups and groups >= leaves and leaves > 1 and plan != torch_ops.PLAN_FLAT:
            groups = 1
        got = _gpu(a, b, op, plan, groups)
        assert got.tobytes() == want.tobytes(), "plan %d groups %d" % (plan, groups)


@pytest.mark.parametrize("opname", ["NN", "NT", "TN"])
def test_public_call_with_host_buffers(opname):
    op = OPS[opname]
    a, b = _operands(70, 90, 640, op, 1)
    got = linalg.matmul(a, b, transpose_a=(opname == "TN"), transpose_b=(opname == "NT"))
    assert got.tobytes() == oracle.nan_canon(oracle.gemm(a, b, op)).tobytes()
    out = np.full((70, 90), -987654.0, np.float32)  # poison: an unwritten cell would survive
    ret = linalg.matmul(a, b, transpose_a=(opname == "TN"), transpose_b=(opname == "NT"), out=out)
    assert ret is out and out.tobytes() == got.tobytes()


@pytest.mark.parametrize("opname", ["NN", "NT"])
def test_host_call_tall_operand_is_pipelined_in_row_chunks(opname):
    """m >= 1024 with host buffers: the rows of A cross in chunks while earlier chunks are multiplied and their
    rows of C return; every chunk is a product of its own, so the bits are the whole product's."""
    op = OPS[opname]
    m, n, k = 1100, 300, 264  # three chunks (384 + 384 + 332 rows), ragged tiles, three leaves with a short last one
    a, b = _operands(m, n, k, op, 5)
    a[7, ::5] = np.float32(1e-41)
    want = oracle.nan_canon(oracle.gemm_rows(a, b, op))
    got = linalg.matmul(a, b, transpose_b=(op == oracle.OP_NT))
    assert got.tobytes() == want.tobytes()
    again = linalg.matmul(a, b, transpose_b=(op == oracle.OP_NT))  # the pooled buffers and events are reused
    assert again.tobytes() == want.tobytes()
    if op == oracle.OP_NT:
        rng = np.random.default_rng(6)
        codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
        exps = rng.integers(-9, -5, n).astype(np.int32)
        want8 = oracle.gemm_rows(a, oracle.dequantize_int8(codes, exps), oracle.OP_NT)
        assert linalg.matmul_int8w(a, codes, exps).tobytes() == want8.tobytes()
    assert _native.lib().b200i_decode_status(-1) == 0


def test_host_call_wide_weight_is_pipelined_in_column_chunks():
    """A short left operand against a wide k-contiguous weight with host buffers: the weight crosses in row chunks,
    each chunk's columns of C are computed densely and return through a strided copy."""
    m, n, k = 40, 2300, 136  # four chunks (640 + 640 + 640 + 380 weight rows), two leaves with a short last one
    a, b = _operands(m, n, k, oracle.OP_NT, 9)
    b[5, ::3] = np.float32(1e-41)
    want = oracle.nan_canon(oracle.gemm_rows(a, b, oracle.OP_NT))
    for _ in range(2):  # the pooled buffers and events are reused
        assert linalg.matmul(a, b, transpose_b=True).tobytes() == want.tobytes()
    rng = np.random.default_rng(10)
    codes = rng.integers(-127, 128, (n, k)).astype(np.int8)
    exps = rng.integers(-9, -5, n).astype(np.int32)
    want8 = oracle.gemm_rows(a, oracle.dequantize_int8(codes, exps), oracle.OP_NT)
    assert linalg.matmul_int8w(a, codes, exps).tobytes() == want8.tobytes()
    bits = oracle.to_bf16((b * 0.02).astype(np.float32))
    wantb = oracle.gemm_rows(a, oracle.from_bf16(bits), oracle.OP_NT)
    assert linalg.matmul_bf16(a, bits, transpose_b=True).tobytes() == wantb.tobytes()
    assert _native.lib().b200i_decode_status(-1) == 0


def test_subnormal_forcing_operands_take_the_flushed_path():
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((150, 300)) * 2.0 ** -62).astype(np.float32)
    b = (rng.standard_normal((300, 140)) * 2.0 ** -63).astype(np.float32)
    a[::3, ::7] = np.float32(1e-41)  # subnormal operands
    b[::5, ::3] = -0.0
    want = oracle.gemm(a, b)
    assert ((want != 0) & (np.abs(want) < 2.0 ** -118)).any()
    for plan, groups in PLANS:
        assert _gpu(a, b, oracle.OP_NN, plan, min(groups, 2)).tobytes() == want.tobytes()
    # the boundary window: exact values in [2^-126 - 2^-150, 2^-126) round up and are kept
    a2 = np.full((4, 130), np.float32(1.0) - np.float32(2.0 ** -24), np.float32)
    b2 = np.zeros((130, 4), np.float32)
    b2[0, :] = np.float32(2.0 ** -126)
    want2 = oracle.gemm(a2, b2)
    assert (want2.view(np.uint32) == 0x00800000).all()
    for plan, groups in PLANS:
        assert _gpu(a2, b2, oracle.OP_NN, plan, min(groups, 1)).tobytes() == want2.tobytes()


def test_signed_zero_nan_and_inf():
    a = np.zeros((5, 300), np.float32)
    a[:] = -0.0
    b = np.ones((300, 6), np.float32)
    want = oracle.gemm(a, b)
    assert not np.signbit(want).any()
    assert _gpu(a, b, oracle.OP_NN).tobytes() == want.tobytes()
    rng = np.random.default_rng(1)
    a = rng.standard_normal((33, 260)).astype(np.float32)
    b = rng.standard_normal((260, 65)).astype(np.float32)
    a[3, 5] = np.nan
    a[7, 200] = np.inf
    b[100, 9] = -np.inf
    want = oracle.nan_canon(oracle.gemm(a, b))
    for plan, groups in PLANS:
        got = _gpu(a, b, oracle.OP_NN, plan, min(groups, 2))
        assert got.tobytes() == want.tobytes()
    assert (want.view(np.uint32)[np.isnan(want)] == 0x7FC00000).all()


def test_batch_invariance():
    """One row alone equals that row inside a bigger call; one column likewise (n: 4 vs 4096)."""
    rng = np.random.default_rng(2)
    a = rng.standard_normal((300, 1000)).astype(np.float32)
    b = rng.standard_normal((4096, 1000)).astype(np.float32)
    full = _gpu(a, b, oracle.OP_NT)
    for i in (0, 7, 299):
        assert _gpu(a[i:i + 1].copy(), b, oracle.OP_NT).tobytes() == full[i:i + 1].tobytes()
    assert _gpu(a, b[:4].copy(), oracle.OP_NT).tobytes() == np.ascontiguousarray(full[:, :4]).tobytes()
    assert _gpu(a[:8].copy(), b, oracle.OP_NT).tobytes() == full[:8].tobytes()


def test_tail_shape_1000_cubed_against_cpu_rows():
    rng = np.random.default_rng(0)
    a = rng.standard_normal((1000, 1000)).astype(np.float32)
    b = rng.standard_normal((1000, 1000)).astype(np.float32)
    want = oracle.gemm_rows(a, b, oracle.OP_NN)
    assert _gpu(a, b, oracle.OP_NN).tobytes() == want.tobytes()
    assert _gpu(a, b, oracle.OP_NT).tobytes() == oracle.gemm_rows(a, b, oracle.OP_NT).tobytes()


def test_config1_1024_cubed_uniform_seed0():
    """The reference's CPU-runnable benchmark case: M = N = K = 1024, U(-1, 1) from seed 0, bit for bit."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1.0, 1.0, (1024, 1024)).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, (1024, 1024)).astype(np.float32)
    want = oracle.gemm_rows(a, b, oracle.OP_NN)
    got = linalg.matmul(a, b)
    assert got.tobytes() == want.tobytes()
    assert oracle.gemm(a[:8], b).tobytes() == want[:8].tobytes()  # the scalar oracle on a sample of rows


@pytest.mark.parametrize("m,n,k", [(4096, 4096, 4096), (8192, 8192, 1024), (128, 11008, 4096), (2048, 50304, 768),
                                   (1000, 1000, 1000)])
def test_config2_full_size_whole_output_against_the_oracle(m, n, k):
    """The full sizes of the headline benchmark shapes: EVERY cell of the product against the CPU oracle's threaded
    form (which tests/test_oracle_rows.py holds to the scalar oracle), then the plans against each other on the full
    output. Plan-against-plan equality alone could not see an error that every plan shares (the group fold, the
    NaN canonicalisation, the store)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), generator=g, device="cuda", dtype=torch.float32)
    b = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32)
    c = torch_ops.matmul(a, b, transpose_b=True)
    want = oracle.gemm_rows(a.cpu().numpy(), b.cpu().numpy(), oracle.OP_NT)
    assert c.cpu().numpy().tobytes() == want.tobytes()
    del want
    other = torch_ops.product(a, b, None, linalg.W_F32, oracle.OP_NT, plan=torch_ops.PLAN_T64,
                              group_leaves=2 if k >= 256 else 0)
    assert torch.equal(c.view(torch.int32), other.view(torch.int32))
    del other
    for plan in (torch_ops.PLAN_T128, torch_ops.PLAN_PACKED):  # the automatic choice is one of these; both must agree
        other = torch_ops.product(a, b, None, linalg.W_F32, oracle.OP_NT, plan=plan)
        assert torch.equal(c.view(torch.int32), other.view(torch.int32)), plan
        del other
    assert _native.lib().b200i_decode_status(-1) == 0
    if m * n * k <= 128 * 11008 * 4096:
        bt = b.t().contiguous()
        nn = torch_ops.matmul(a, bt)
        assert torch.equal(c.view(torch.int32), nn.view(torch.int32))  # orientations agree


FOLD_PLANS = [torch_ops.PLAN_T128, torch_ops.PLAN_T64, torch_ops.PLAN_T32, torch_ops.PLAN_PACKED, torch_ops.PLAN_SKINNY]


def _fold_sweep_counts():
    rng = np.random.default_rng(2049)
    return list(range(1, 65)) + sorted(set(int(v) for v in rng.integers(65, 1025, 40)))


@pytest.mark.parametrize("chunk", range(8))
def test_fold_over_every_leaf_count(chunk):
    """The streaming fold against the oracle's tree for every leaf count P in 1..64 and 40 random P up to 1024
    (the reference sweeps its stack fold over every P in 1..2049, gemm/checks/gemm_device_check.mojo:284): a 3 x 3
    product, every plan that keeps a fold stack, unsplit and in leaf groups of 1, 2 and 4 (a ragged last group
    included), a short last leaf on the odd counts. Operands of mixed magnitude make every addition order visible."""
    counts = _fold_sweep_counts()[chunk::8]
    for p in counts:
        k = (p - 1) * 128 + (128 if p % 2 == 0 else 48)  # a multiple of 16 so that the skinny and decode plans accept it
        assert oracle.leaf_count(k) == p
        rng = np.random.default_rng(p)
        a = (rng.standard_normal((3, k)) * np.exp2(rng.integers(-12, 13, (3, k)))).astype(np.float32)
        b = (rng.standard_normal((3, k)) * np.exp2(rng.integers(-12, 13, (3, k)))).astype(np.float32)
        want = oracle.nan_canon(oracle.gemm(a, b, oracle.OP_NT))
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        got = {}
        for plan in FOLD_PLANS:
            for groups in (0, 1, 2, 4):
                if groups and (p + groups - 1) // groups > 64:
                    continue  # more leaf groups than a launch takes
                got[(plan, groups)] = torch_ops.product(da, db, None, linalg.W_F32, oracle.OP_NT, plan=plan, group_leaves=groups)
        if _native.lib().b200i_decode_plan_fits(3, 3, k, oracle.OP_NT, linalg.W_F32):
            got[(torch_ops.PLAN_DECODE, 0)] = torch_ops.product(da, db, None, linalg.W_F32, oracle.OP_NT, plan=torch_ops.PLAN_DECODE)
        got[(torch_ops.PLAN_AUTO, 0)] = torch_ops.product(da, db, None, linalg.W_F32, oracle.OP_NT)
        for key, c in got.items():
            assert c.cpu().numpy().tobytes() == want.tobytes(), (p, k) + key
    assert _native.lib().b200i_decode_status(-1) == 0


def test_c_abi_refusals_on_device():
    a = torch.zeros((4, 4), device="cuda")
    with pytest.raises(ValueError):
        torch_ops.product(a, a, None, linalg.W_F32, 7)
    buf = ctypes.create_string_buffer(256)
    rc = _native.lib().b200i_gemm_f32(0, None, a.data_ptr(), a.data_ptr(), a.data_ptr(), 4, 4, 4, 7, None, 0,
                                      ctypes.cast(buf, ctypes.c_void_p), 256)
    assert rc == 1 and b"unknown op" in buf.value
    rc = _native.lib().b200i_gemm_f32(0, None, a.data_ptr(), a.data_ptr(), a.data_ptr(), 0, 4, 4, 0, None, 0,
                                      ctypes.cast(buf, ctypes.c_void_p), 256)
    assert rc == 1 and b"must be positive" in buf.value
    with pytest.raises(TypeError):
        torch_ops.product(a.double(), a)
    with pytest.raises(ValueError):
        torch_ops.product(a.t(), a)
    with pytest.raises(_native.NativeError):
        torch_ops.product(a, a.to(torch.int8), None, linalg.W_INT8_EXP, oracle.OP_NT)


def test_custom_op_registration():
    a = torch.randn((8, 300), device="cuda")
    b = torch.randn((300, 5), device="cuda")
    c = torch.ops.mojolearn_b200.matmul(a, b, 0)
    want = oracle.gemm(a.cpu().numpy(), b.cpu().numpy())
    assert c.cpu().numpy().tobytes() == want.tobytes()


def _seams_after(c, bias, act):
    """The oracle's words of the product followed by the separate bias and activation seams."""
    out = np.array(c, copy=True)
    if bias is not None:
        out = np.vectorize(lambda v, b: oracle.ftz(np.float32(oracle.ftz(v)) + np.float32(oracle.ftz(b))), otypes=[np.float32])(out, bias[None, :])
    name = {0: None, 1: "gelu_erf", 2: "gelu_tanh", 3: "siluf"}[act]
    if name:
        out = np.vectorize(lambda v: oracle.ftz(oracle.math(name, oracle.ftz(v))), otypes=[np.float32])(out)
    return out.astype(np.float32)


@pytest.mark.parametrize("m,n,k", [(9, 20, 300), (5, 131, 640), (40, 70, 129), (3, 64, 2048)])
def test_store_epilogue_bias_and_activation_on_every_plan(m, n, k):
    """GEMM_EPI_PLUS_BIAS / GEMM_EPI_BIAS_ACT (reference gemm/checks/gemm_identical.mojo:8869-8912): the bias add and
    the ungated activation inside the product's store give the words of the product followed by the separate seams,
    on every plan, split and unsplit (a split plan applies them in the group fold, never to a node)."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    a[0, :] = 0.0  # a zero row: the word is the bias (or its activation) alone
    c = oracle.nan_canon(oracle.gemm(a, b, oracle.OP_NT))
    da, db, dbias = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(bias).cuda()
    leaves = oracle.leaf_count(k)
    plans = [(torch_ops.PLAN_AUTO, 0), (torch_ops.PLAN_FLAT, 0), (torch_ops.PLAN_T128, 0), (torch_ops.PLAN_T64, 2), (torch_ops.PLAN_T32, 1),
             (torch_ops.PLAN_PACKED, 0), (torch_ops.PLAN_PACKED, 2), (torch_ops.PLAN_SKINNY, 0), (torch_ops.PLAN_SKINNY, 1)]
    if k % 16 == 0 and m <= 8:
        plans.append((torch_ops.PLAN_DECODE, 0))
    for use_bias, act in ((True, 0), (True, 1), (True, 2), (False, 3), (True, 3), (False, 1)):
        want = _seams_after(c, bias if use_bias else None, act)
        for plan, groups in plans:
            if plan == torch_ops.PLAN_SKINNY and k % 16:
                continue
            if groups and groups >= leaves:
                groups = 0
            got = torch_ops.product(da, db, None, linalg.W_F32, oracle.OP_NT, plan=plan, group_leaves=groups,
                                    bias=dbias if use_bias else None, act=act)
            assert got.cpu().numpy().tobytes() == want.tobytes(), (use_bias, act, plan, groups)
    codes, exps = oracle.quantize_int8(b)
    c8 = oracle.nan_canon(oracle.gemm(a, oracle.dequantize_int8(codes, exps), oracle.OP_NT))
    got = torch_ops.product(da, torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda(), linalg.W_INT8_EXP, oracle.OP_NT, bias=dbias, act=1)
    assert got.cpu().numpy().tobytes() == _seams_after(c8, bias, 1).tobytes()


@pytest.mark.parametrize("m,n,k", [(9, 20, 304), (32, 132, 640), (1, 64, 2048), (3, 8, 128)])
def test_gated_store_activation_over_interleaved_rows(m, n, k):
    """The gated activations (S20-S21: silu(gate) * up, and GELU in SiLU's place) inside the store of a product whose
    weight rows alternate gate_j, up_j: the output [m, n / 2] is the words of the product followed by the separate
    activation seam, on the skinny plan unsplit and split (the group fold applies it), with and without a bias."""
    rng = np.random.default_rng(m * 1000 + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    c = oracle.nan_canon(oracle.gemm(a, w, oracle.OP_NT))
    da, dw, dbias = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda()
    leaves = oracle.leaf_count(k)
    ftz, f32 = oracle.ftz, np.float32
    for use_bias in (False, True):
        cb = np.vectorize(lambda v, b: ftz(f32(ftz(v)) + f32(ftz(b))), otypes=[np.float32])(c, bias[None, :]) if use_bias else c
        for act, name in ((4, "siluf"), (5, "gelu_erf"), (6, "gelu_tanh")):
            gate, up = cb[:, 0::2], cb[:, 1::2]
            want = np.vectorize(lambda g, u: ftz(f32(ftz(oracle.math(name, ftz(g)))) * f32(ftz(u))), otypes=[np.float32])(gate, up)
            for plan, groups in ((torch_ops.PLAN_AUTO, 0), (torch_ops.PLAN_SKINNY, 0), (torch_ops.PLAN_SKINNY, 1), (torch_ops.PLAN_SKINNY, 2)):
                if groups and groups >= leaves:
                    continue
                got = torch_ops.product(da, dw, None, linalg.W_F32, oracle.OP_NT, plan=plan, group_leaves=groups,
                                        bias=dbias if use_bias else None, act=act)
                assert got.shape == (m, n // 2) and got.cpu().numpy().tobytes() == want.tobytes(), (use_bias, act, plan, groups)
            # the same seam as its own kernel over the interleaved product
            full = torch_ops.product(da, dw, None, linalg.W_F32, oracle.OP_NT, bias=dbias if use_bias else None)
            out = torch.empty((m, n // 2), device="cuda")
            _native.call("b200i_act_mul", 0, None, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(full.data_ptr()), None, m, n // 2, n,
                         {4: 0, 5: 4, 6: 5}[act], 1)
            assert out.cpu().numpy().tobytes() == want.tobytes()
    codes, exps = oracle.quantize_int8(w)
    c8 = oracle.nan_canon(oracle.gemm(a, oracle.dequantize_int8(codes, exps), oracle.OP_NT))
    want8 = np.vectorize(lambda g, u: ftz(f32(ftz(oracle.math("siluf", ftz(g)))) * f32(ftz(u))), otypes=[np.float32])(c8[:, 0::2], c8[:, 1::2])
    got8 = torch_ops.product(da, torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda(), linalg.W_INT8_EXP, oracle.OP_NT, act=4)
    assert got8.cpu().numpy().tobytes() == want8.tobytes()
    with pytest.raises(_native.NativeError, match="gated store activation"):
        torch_ops.product(torch.zeros((40, 64), device="cuda"), torch.zeros((8, 64), device="cuda"), None, linalg.W_F32, oracle.OP_NT, act=4)

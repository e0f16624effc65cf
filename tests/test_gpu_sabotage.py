"""Negative control for the admission test (the reference pairs every gate with a sabotage arm that must fail:
gemm/checks/gemm_identical.mojo:229-271, MOJOLEARN_GEMM_SABOTAGE_ADMIT_ALWAYS :1444, checks/kernel_matrix_gemm.mojo:124-134).

A second build of the CUDA library admits every window to the bare multiply-add, whatever its operands. Loaded in a
child process through MOJOLEARN_B200_LIB, it must get the subnormal-forcing products and a subnormal-forcing attention
call WRONG (other bits only: nothing faults), and still get an ordinary product right. That is what shows that the
same cases, green on the real library, would catch a broken admission test.
"""
import json
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys
sys.path[:0] = [%(root)r, %(root)r + "/tests", %(root)r + "/tests/golden"]
import numpy as np, torch
import oracle, decoder_ref, fixtures
from mojolearn_b200 import _native, linalg, torch_ops
rng = np.random.default_rng(0)
a = (rng.standard_normal((150, 300)) * 2.0 ** -62).astype(np.float32)
b = (rng.standard_normal((300, 140)) * 2.0 ** -63).astype(np.float32)
a[::3, ::7] = np.float32(1e-41)
want = oracle.gemm(a, b)
out = {"lib": _native.LIB_PATH, "plans": {}}
da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
for name, plan in (("flat", torch_ops.PLAN_FLAT), ("t128", torch_ops.PLAN_T128), ("t64", torch_ops.PLAN_T64), ("t32", torch_ops.PLAN_T32),
                   ("packed", torch_ops.PLAN_PACKED), ("auto", torch_ops.PLAN_AUTO)):
    got = torch_ops.product(da, db, None, linalg.W_F32, oracle.OP_NN, plan=plan).cpu().numpy()
    out["plans"][name] = got.tobytes() == want.tobytes()
x = rng.standard_normal((9, 300)).astype(np.float32)
w = rng.standard_normal((20, 300)).astype(np.float32)
out["ordinary"] = linalg.matmul(x, w, transpose_b=True).tobytes() == oracle.gemm(x, w, oracle.OP_NT).tobytes()
xs = (rng.standard_normal((8, 256)) * 2.0 ** -62).astype(np.float32)
ws = (rng.standard_normal((300, 256)) * 2.0 ** -63).astype(np.float32)
codes, exps = oracle.quantize_int8(ws)
w8 = oracle.dequantize_int8(codes, exps)
got = torch_ops.product(torch.from_numpy(xs).cuda(), torch.from_numpy(codes).cuda(), torch.from_numpy(exps).cuda(), linalg.W_INT8_EXP, oracle.OP_NT,
                        plan=torch_ops.PLAN_SKINNY).cpu().numpy()
out["skinny_int8"] = got.tobytes() == oracle.gemm(xs, w8, oracle.OP_NT).tobytes()
# a prompt-sized attention call whose value rows sit near 2^-124: every weighted value is subnormal, so the flushed
# chain leaves exact zeros where the bare chain piles up a normal number
import ctypes
bq, l, nh, hd = 1, 200, 2, 64
q = (rng.standard_normal((bq * l, nh, hd)) * 0.3).astype(np.float32)
kc = rng.standard_normal((bq, nh, l, hd)).astype(np.float32)
vc = (rng.standard_normal((bq, nh, l, hd)) * 2.0 ** -124).astype(np.float32)
dq, dk, dv = (torch.from_numpy(t).cuda() for t in (q, kc, vc))
ctx = torch.empty((bq * l, nh * hd), device="cuda")
scores = torch.empty((bq * nh * l * l,), device="cuda")
vp = lambda t: ctypes.c_void_p(t.data_ptr())
_native.call("b200i_attention", 0, None, vp(ctx), vp(dq), vp(dk), vp(dv), vp(scores), bq, l, nh, nh, hd, l, l, 0, 0.0)
out["attention"] = ctx.cpu().numpy().tobytes() == oracle.attention(q, kc, vc, l, l).tobytes()
torch.cuda.synchronize()
print("RESULT " + json.dumps(out))
"""


def _child(lib=None):
    env = dict(os.environ)
    env.pop("MOJOLEARN_B200_LIB", None)
    if lib:
        env["MOJOLEARN_B200_LIB"] = lib
    run = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-3000:]
    line = [ln for ln in run.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_admit_always_build_fails_the_subnormal_forcing_cases():
    from mojolearn_b200.csrc import build as cuda_build
    sabotage = cuda_build.build(sabotage=True)
    real = _child()
    assert real["lib"].endswith("libb200i.so")
    assert all(real["plans"].values()) and real["ordinary"] and real["skinny_int8"] and real["attention"], real
    bad = _child(sabotage)
    assert bad["lib"] == sabotage
    assert bad["ordinary"], "the sabotaged build must still get ordinary operands right"
    assert bad["plans"]["flat"], "the flat plan flushes every step and has no admission test to break"
    for plan in ("t128", "t64", "t32", "packed", "auto"):
        assert not bad["plans"][plan], "plan %s passed the subnormal-forcing product with admission sabotaged" % plan
    assert not bad["skinny_int8"], "the register skinny plan passed with admission sabotaged"
    assert not bad["attention"], "the subnormal-forcing attention call passed with admission sabotaged"

"""A bounded device-side wait that ran out must never return as a silent success.

The kernels record such a wait in one device status word and skip their stores. These tests write that word from the
host (b200i_debug_set_status; no kernel is made to time out) and check that every synchronous door reports it: the
host-pointer twins return status 1 with a message (the reference's status + message buffer,
adapters/native/c_api.mojo:64-72), `torch_ops.check_status`, `CausalLM.generate` and the decode sessions raise, and
the word is cleared by the report.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mojolearn_b200 import _native, linalg, torch_ops  # noqa: E402
from mojolearn_b200.models import CausalLM, CausalLMConfig  # noqa: E402

import decoder_ref  # noqa: E402


def _set(value):
    assert _native.lib().b200i_debug_set_status(0, value) == 0


def test_host_twins_report_a_wait_that_ran_out():
    rng = np.random.default_rng(0)
    a = rng.standard_normal((8, 64)).astype(np.float32)
    w = rng.standard_normal((16, 64)).astype(np.float32)
    want = linalg.matmul(a, w, transpose_b=True)
    _set(5)
    with pytest.raises(_native.NativeError, match="wait ran out.*status 5"):
        linalg.matmul(a, w, transpose_b=True)
    assert _native.lib().b200i_decode_status(0) == 0  # cleared by the report
    assert linalg.matmul(a, w, transpose_b=True).tobytes() == want.tobytes()
    _set(2)
    with pytest.raises(_native.NativeError, match="status 2"):
        linalg.to_bf16(a)
    big_a = rng.standard_normal((1024, 256)).astype(np.float32)  # the pipelined host path
    big_w = rng.standard_normal((256, 256)).astype(np.float32)
    _set(4)
    with pytest.raises(_native.NativeError, match="status 4"):
        linalg.matmul(big_a, big_w, transpose_b=True)
    linalg.matmul(big_a, big_w, transpose_b=True)


def test_device_callers_report_it_at_their_synchronise():
    _set(1)
    with pytest.raises(_native.NativeError, match="status 1"):
        torch_ops.check_status(torch.device("cuda", 0))
    torch_ops.check_status(torch.device("cuda", 0))
    cfg = CausalLMConfig(vocab=31, d_model=16, n_layers=1, n_heads=2, head_dim=8, intermediate=32, max_positions=32)
    lm = CausalLM(cfg, decoder_ref.random_lm_weights(cfg, seed=1, scale=0.2))
    ids = np.random.default_rng(1).integers(0, cfg.vocab, (2, 4)).astype(np.int32)
    seq = lm.generate(ids, 3)
    _set(3)
    with pytest.raises(_native.NativeError, match="status 3"):
        lm.generate(ids, 3)
    assert lm.generate(ids, 3).tolist() == seq.tolist()
    _set(8)
    with pytest.raises(_native.NativeError, match="status 8"):
        lm.forward(ids)
    state = lm.allocate_state(2, 8)
    session = lm.decode_session(state, lm.forward_device(ids, state, last_only=True))
    session.step()
    _set(7)
    with pytest.raises(_native.NativeError, match="status 7"):
        session.check_status()
    session.check_status()

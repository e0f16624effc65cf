"""Output-column sharded serving on 2 GPUs: logits and greedy ids bit-identical to the
single-GPU run, with the decode-step gathers through the store-side peer exchange and
through the NCCL all-gather, and with the prompt cut by sequences and by output columns.
Skipped with fewer than 2 devices."""
import json
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ARGS = ["--layers", "2", "--d-model", "512", "--heads", "8", "--mlp", "1024", "--vocab", "4096", "--batch", "4", "--prompt", "24",
        "--decode", "6", "--timed-steps", "3"]


def _run(cmd, **extra):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra)
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    if out.returncode != 0:
        lines = out.stderr.splitlines()
        culprit = [i for i, ln in enumerate(lines) if "Error" in ln and "ChildFailedError" not in ln]
        at = culprit[0] if culprit else max(0, len(lines) - 40)
        raise AssertionError("\n".join(lines[max(0, at - 25):at + 5]))
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_serving_equals_single_gpu():
    one = _run([sys.executable, "-m", "mojolearn_b200.serve_bench"] + ARGS)
    # the last variant injects a host-side failure into rank 1's exchange set-up: every rank must then agree to fall back
    variants = (dict(), dict(MOJOLEARN_B200_EXCHANGE="0"), dict(MOJOLEARN_B200_PREFILL="columns"), dict(MOJOLEARN_B200_EXCHANGE_FAIL_RANK="1"))
    for i, extra in enumerate(variants):
        launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                  "--master-port", str(29517 + i), "-m", "mojolearn_b200.serve_bench"] + ARGS  # a port of its own: the last run's may linger
        two = _run(launch, **extra)
        assert two["n_gpus"] == 2, extra
        assert one["ids_sha256"] == two["ids_sha256"] and one["logits_sha256"] == two["logits_sha256"], extra
        nccl = extra.get("MOJOLEARN_B200_EXCHANGE") == "0" or "MOJOLEARN_B200_EXCHANGE_FAIL_RANK" in extra
        assert two["config"]["gathers"] == ("NCCL all-gather" if nccl else "peer stores"), extra

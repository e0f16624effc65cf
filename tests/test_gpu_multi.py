"""Output-column sharded serving on 2 GPUs (NCCL all-gather): logits and greedy
ids bit-identical to the single-GPU run. Skipped with fewer than 2 devices."""
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


def _run(cmd):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_serving_equals_single_gpu():
    one = _run([sys.executable, "-m", "mojolearn_b200.serve_bench"] + ARGS)
    two = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                "--master-port", "29517", "-m", "mojolearn_b200.serve_bench"] + ARGS)
    assert two["n_gpus"] == 2
    assert one["ids_sha256"] == two["ids_sha256"] and one["logits_sha256"] == two["logits_sha256"]

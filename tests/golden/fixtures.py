"""The nine seeded fixtures the reference's verify table is recorded on, and
the GEMM identity card's shape table, regenerated locally.

These follow tools/identity_break.py:1393-1471 (`fixture`, `_hashed_uniform`)
and bench/gemm_shapes.mojo:153-274 / bench/gemm_card_main.mojo:361-378 of the
reference. The generators are numpy's PCG64 `default_rng` and sha256, so the
bytes are reproducible here; the verify table carries a hash of each fixture,
which tests/test_oracle_golden.py checks before it trusts any product hash.
"""
import hashlib

import numpy as np

N_ROWS, N_COLS = 20000, 16
KINDS = ["base", "ties", "hashed", "wide", "denormal", "denormal_ftz", "dupes", "odd", "negative"]


def _sha_stream_uniform(n, d, seed):
    ctr = np.arange(n * d, dtype=np.uint64)
    dig = hashlib.sha256(ctr.tobytes() + str(seed).encode()).digest()
    need = n * d * 4
    chunks, blk, have = [], 0, 0
    while have < need:
        h = hashlib.sha256(dig + blk.to_bytes(8, "little")).digest()
        chunks.append(h)
        have += len(h)
        blk += 1
    u32 = np.frombuffer(b"".join(chunks)[:need], dtype=np.uint32)
    return (u32.astype(np.float64) / 2 ** 32).astype(np.float32).reshape(n, d)


def fixture(kind, seed=0, n=N_ROWS, d=N_COLS):
    rng = np.random.default_rng(seed)
    if kind == "base":
        return rng.standard_normal((n, d)).astype(np.float32)
    if kind == "ties":
        return rng.integers(0, 6, size=(n, d)).astype(np.float32)
    if kind == "hashed":
        return (_sha_stream_uniform(n, d, seed) * 4.0 - 2.0).astype(np.float32)
    if kind == "wide":
        x = rng.standard_normal((n, d)).astype(np.float32)
        return (x * np.logspace(-4, 4, d).astype(np.float32)).astype(np.float32)
    if kind == "denormal":
        x = rng.standard_normal((n, d)).astype(np.float32)
        x[: n // 4, :3] = (x[: n // 4, :3] * np.float32(1e-40)).astype(np.float32)
        return x
    if kind == "denormal_ftz":
        x = fixture("denormal", seed, n, d).copy()
        sub = (x != 0) & (np.abs(x) < np.finfo(np.float32).tiny)
        x[sub] = np.copysign(np.float32(0.0), x[sub])
        return x
    if kind == "dupes":
        x = rng.standard_normal((n, d)).astype(np.float32)
        x[n // 2:] = x[: n - n // 2]
        x[:, d - 2] = np.float32(3.5)
        x[:, d - 1] = np.float32(0.0)
        return x
    if kind == "odd":
        return rng.standard_normal((12345, 17)).astype(np.float32)
    if kind == "negative":
        return (-np.abs(rng.standard_normal((n, d))) - 2.0).astype(np.float32)
    raise ValueError(kind)


# The identity card's 20 shapes: (name, table op, m, n, k). Rows 0-3 are TN, the
# rest NT (bench/gemm_shapes.mojo:153-274).
CARD_SHAPES = [
    ("gram.32x32x1M", "TN", 32, 32, 1_000_000),
    ("gram.32x32x64K", "TN", 32, 32, 65_536),
    ("gram.128sq.x100003", "TN", 128, 128, 100_003),
    ("ols.step1.16x16x64K", "TN", 16, 16, 65_536),
    ("pca.transform.8192x4x4", "NT", 8192, 4, 4),
    ("pca.transform.wide.8192x64x128", "NT", 8192, 64, 128),
    ("kmeans.dist.4096x64x64", "NT", 4096, 64, 64),
    ("ols.predict.gemv.64Kx16", "NT", 65536, 1, 16),
    ("llama8b.qkv.t1", "NT", 1, 4096, 4096),
    ("llama8b.qkv.t8", "NT", 8, 4096, 4096),
    ("llama8b.qkv.t512", "NT", 512, 4096, 4096),
    ("llama8b.mlp_up.t1", "NT", 1, 14336, 4096),
    ("llama8b.mlp_up.t8", "NT", 8, 14336, 4096),
    ("llama8b.mlp_up.t512", "NT", 512, 14336, 4096),
    ("llama8b.mlp_down.t1", "NT", 1, 4096, 14336),
    ("llama8b.mlp_down.t8", "NT", 8, 4096, 14336),
    ("llama8b.mlp_down.t512", "NT", 512, 4096, 14336),
    ("llama8b.lm_head.t1", "NT", 1, 128256, 4096),
    ("llama8b.lm_head.t8", "NT", 8, 128256, 4096),
    ("llama8b.lm_head.t512", "NT", 512, 128256, 4096),
]

HOST_MAC_BUDGET = 16_000_000


def card_capped(m, n, k):
    """m and n halved (the larger first) until m*n*k fits the card's host
    budget; k is never touched (bench/gemm_card_main.mojo:361-378)."""
    while m * n * k > HOST_MAC_BUDGET and (m > 1 or n > 1):
        if n >= m and n > 1:
            n = (n + 1) // 2
        elif m > 1:
            m = (m + 1) // 2
        else:
            break
    return m, n


def card_operands(index, fill):
    """Shapes and fills of card row `index`. `fill(count, salt)` returns the
    flat float32 values (salts 11+i and 22+i, bench/gemm_card_main.mojo:682-692).
    Returns (name, op_name, a, b) with a and b shaped for that op."""
    name, op, m0, n0, k = CARD_SHAPES[index]
    m, n = card_capped(m0, n0, k)
    if op == "TN":
        a = fill(k * m, 11 + index).reshape(k, m)
        b = fill(k * n, 22 + index).reshape(k, n)
    else:
        a = fill(m * k, 11 + index).reshape(m, k)
        b = fill(n * k, 22 + index).reshape(n, k)
    return name, op, a, b

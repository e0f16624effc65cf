"""Bit-neutral sharding of a linear layer across one process per GPU.

A cell C[i, j] of the identical-mode product reads row i of the activations and
row j of the weight and nothing else, and its bits depend on k and the profile
alone (reference gemm/IDENTICAL_FP32_CONTRACT.md:112-116). So the only axes a
layer may be cut along are output columns (weight rows) and batch; k is never
split and nothing is ever all-reduced, because a k split is a summation order.
Rank r keeps weight rows [r*N/g, (r+1)*N/g), computes its column slice with the
full k, and the slices are concatenated by an all-gather, which moves finished
float32 words and performs no arithmetic. The reference's own multi-device rule
is the same: byte copies only, never a collective that picks an order
(training/byte_lm_parallel.py:2-8, core/multi_gpu.mojo:2-6).
"""
import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """Rows [lo, hi) of an n-row weight owned by `rank`; n must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d outside a world of %d" % (rank, world))
    if n % world:
        raise ValueError("%d output columns do not divide over %d ranks" % (n, world))
    return rank * n // world, (rank + 1) * n // world


def gather_columns(part, group=None):
    """[m, n/g] column slices on every rank -> the full [m, n] on every rank (rank order = column order)."""
    world = dist.get_world_size(group)
    if world == 1:
        return part
    part = part.contiguous()
    m, w = part.shape
    gathered = torch.empty((world * m, w), dtype=part.dtype, device=part.device)  # rank-major concatenation
    dist.all_gather_into_tensor(gathered, part, group=group)
    return gathered.view(world, m, w).permute(1, 0, 2).reshape(m, world * w).contiguous()

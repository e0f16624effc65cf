"""The fold SCHEDULES the CUDA kernels use, restated on the host and held to the oracle's balanced tree (adjacent
pairs, an odd tail carried up; `oracle.fold`): the binary-counter stack every product kernel streams its leaves
through (a node is pushed, merging while the counter's low bits are set; the last node drains the stack), and the
two-stage form of `fold_groups_split_kernel` and `comm_fold_gather_kernel` (blocks of eight nodes folded separately,
the last block possibly ragged, then the block roots folded the same way three levels up). Float32 addition is not
associative, so equal bits on operands of mixed magnitude mean equal trees; the symbolic check says so exactly."""
import numpy as np
import pytest

import oracle


def counter_fold(nodes, add, levels):
    """fold_push of the CUDA sources: stack[levels], node gi of len(nodes)."""
    stack = [None] * levels
    last = len(nodes) - 1
    for gi, v in enumerate(nodes):
        if gi == last:
            for lvl in range(levels):
                if (last >> lvl) & 1:
                    v = add(stack[lvl], v)
            return v
        for lvl in range(levels):
            if (gi >> lvl) & 1:
                v = add(stack[lvl], v)
            else:
                stack[lvl] = v
                break
        else:
            raise AssertionError("the stack is too shallow for %d nodes" % len(nodes))
    raise AssertionError("no nodes")


def block_fold(nodes, add, sub=8):
    roots = [counter_fold(nodes[g0:g0 + sub], add, 3) for g0 in range(0, len(nodes), sub)]
    return counter_fold(roots, add, 3)


def contract_tree(nodes, add):
    """Adjacent pairs level by level, an odd tail carried unchanged (the contract's fold)."""
    level = list(nodes)
    while len(level) > 1:
        nxt = [add(level[i], level[i + 1]) for i in range(0, len(level) - 1, 2)]
        if len(level) % 2:
            nxt.append(level[-1])
        level = nxt
    return level[0]


def test_schedules_build_the_contract_tree_symbolically():
    pair = lambda a, b: (a, b)  # noqa: E731
    for count in range(1, 65):
        leaves = list(range(count))
        want = contract_tree(leaves, pair)
        assert counter_fold(leaves, pair, 6) == want, count
        assert block_fold(leaves, pair) == want, count
    for count in (65, 100, 255, 256, 257, 1000, 1024):
        leaves = list(range(count))
        assert counter_fold(leaves, pair, 10) == contract_tree(leaves, pair), count


@pytest.mark.parametrize("seed", range(3))
def test_schedules_give_the_oracle_bits(seed):
    rng = np.random.default_rng(seed)
    add = lambda a, b: np.float32(a + b)  # noqa: E731  (normal-range operands: nothing to flush)
    for count in list(range(1, 65)) + [100, 257, 1024]:
        v = (rng.standard_normal(count) * np.exp2(rng.integers(-12, 13, count))).astype(np.float32)
        want = np.float32(oracle.fold(v, "tree"))
        got = counter_fold(list(v), add, 10)
        assert got.tobytes() == want.tobytes(), count
        if count <= 64:
            assert block_fold(list(v), add).tobytes() == want.tobytes(), count

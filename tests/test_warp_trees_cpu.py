"""The in-warp trees of the router kernels (warp_trees32, llmxabe_b200/csrc/glue_kernels.cuh), restated
on the CPU lane by lane and compared bit for bit with the shuffle-down tree they replace.

The reference's router (crates/xabe-engine/src/block/moe.rs:347-368) reduces each group of 32 lanes
with `for (off = 16; off > 0; off >>= 1) v += __shfl_down_sync(full, v, off)` and takes lane 0's value.
warp_trees32 evaluates 32 such trees at once: at the level with offset `half` lanes l and l ^ half swap
halves of the addends they still hold and add what they receive to what they keep.  fp32 addition
rounds, so "the same tree" is a statement about which pairs are added in which order; this test checks
it on random and on cancellation-prone inputs.
"""
import numpy as np


def shuffle_down_tree(v: np.ndarray) -> np.float32:
    """Lane 0 of the shuffle-down tree over 32 lanes (a lane past the end returns the caller's own value)."""
    v = v.astype(np.float32).copy()
    for off in (16, 8, 4, 2, 1):
        src = np.arange(32) + off
        got = np.where(src < 32, v[np.minimum(src, 31)], v)
        v = (v + got).astype(np.float32)
    return v[0]


def warp_trees32(a: np.ndarray) -> np.ndarray:
    """a[lane][o]: lane's addend of output o.  Returns, per lane o, the total of output o."""
    a = a.astype(np.float32).copy()            # [32 lanes][32 values]
    lanes = np.arange(32)
    for half in (16, 8, 4, 2, 1):
        upper = (lanes & half) != 0
        new = np.empty((32, half), dtype=np.float32)
        for i in range(half):
            send = np.where(upper, a[:, i], a[:, half + i])
            keep = np.where(upper, a[:, half + i], a[:, i])
            recv = send[lanes ^ half]          # __shfl_xor_sync(send, half)
            new[:, i] = np.where(upper, (recv + keep).astype(np.float32), (keep + recv).astype(np.float32))
        a = new
    return a[:, 0]


def _check(a: np.ndarray) -> None:
    got = warp_trees32(a)
    for o in range(32):
        want = shuffle_down_tree(a[:, o])
        assert got[o].view(np.uint32) == want.view(np.uint32), (o, got[o], want)


def test_in_warp_trees_equal_the_shuffle_down_tree_bit_for_bit():
    rng = np.random.default_rng(0)
    for _ in range(20):
        _check(rng.standard_normal((32, 32)).astype(np.float32))


def test_in_warp_trees_on_inputs_where_the_order_of_additions_shows():
    rng = np.random.default_rng(1)
    for _ in range(20):
        a = (rng.standard_normal((32, 32)) * 10.0 ** rng.integers(-6, 7, size=(32, 32))).astype(np.float32)
        _check(a)
    # a different pairing would give a different sum here
    a = np.zeros((32, 32), dtype=np.float32)
    a[0, :] = 1.0e8
    a[16, :] = -1.0e8
    a[1, :] = 1.0
    _check(a)
    assert shuffle_down_tree(a[:, 0]) == np.float32(1.0)

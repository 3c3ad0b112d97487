"""Double-tree all-reduce protocol model: W in {2,4,8}, 1,048,576 fp32 from
N(0,1) seeded by rank, 64 chunks alternating between the trees, against the
elementwise sum."""
import numpy as np
import pytest

from tccl_b200 import simulate_double_tree_all_reduce
from tccl_b200.parallel.simulate import chunk_bounds


@pytest.mark.parametrize("W", [2, 4, 8])
def test_config1(W):
    xs = [np.random.default_rng(r).standard_normal(1 << 20).astype(np.float32) for r in range(W)]
    outs = simulate_double_tree_all_reduce(xs, n_chunks=64)
    ref = np.sum(np.stack(xs).astype(np.float64), axis=0)
    for o in outs:
        # rtol 1e-5 as specified; sums close to zero need an absolute floor of a few fp32 ulps of the operands
        np.testing.assert_allclose(o, ref, rtol=1e-5, atol=2e-6)
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])  # every rank holds the same bits


@pytest.mark.parametrize("W", [1, 3, 5, 6, 7])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_other_worlds_and_interleavings(W, seed):
    xs = [np.random.default_rng(10 + r).standard_normal(4099).astype(np.float32) for r in range(W)]
    outs = simulate_double_tree_all_reduce(xs, n_chunks=7, seed=seed)
    ref = np.sum(np.stack(xs).astype(np.float64), axis=0)
    for o in outs:
        np.testing.assert_allclose(o, ref, rtol=1e-5, atol=2e-6)


def test_inputs_untouched_and_bounds():
    xs = [np.ones(100, np.float32) * r for r in range(4)]
    keep = [x.copy() for x in xs]
    simulate_double_tree_all_reduce(xs, n_chunks=3)
    for a, b in zip(xs, keep):
        assert np.array_equal(a, b)
    b = chunk_bounds(100, 8, align=4)
    assert b[0] == (0, 16) and b[-1][1] == 100 and all(lo % 4 == 0 for lo, _ in b)
    assert sum(hi - lo for lo, hi in b) == 100

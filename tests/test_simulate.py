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


@pytest.mark.parametrize("pull_down", [False, True])
@pytest.mark.parametrize("depth", [1, 2, 4])
@pytest.mark.parametrize("W", [2, 3, 5, 8])
def test_ring_flow_control_and_both_ways_down_over_back_to_back_calls(W, depth, pull_down):
    """Partials travel through a ring of `depth` slots per (tree, child) that a child refills only
    after the parent's acknowledgement; the sum comes down pushed or pulled; three calls run on the
    same counters with the ranks free of each other.  Any interleaving must give the sum."""
    xs = [np.random.default_rng(30 + r).standard_normal(1031).astype(np.float32) for r in range(W)]
    ref = np.sum(np.stack(xs).astype(np.float64), axis=0)
    for seed in range(4):
        outs = simulate_double_tree_all_reduce(xs, n_chunks=13, seed=seed, ring_depth=depth, pull_down=pull_down, calls=3)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=1e-5, atol=2e-6)
            assert np.array_equal(o, outs[0])


def test_the_model_notices_a_ring_without_flow_control():
    """Without the ACK wait a fast child overwrites a slot its parent has not read: the model's own
    assertion (the check the other tests rely on) must fire for some interleaving."""
    xs = [np.ones(64, np.float32) * (r + 1) for r in range(4)]
    caught = 0
    for seed in range(20):
        try:
            simulate_double_tree_all_reduce(xs, n_chunks=24, seed=seed, ring_depth=1, wait_for_ack=False)
        except AssertionError:
            caught += 1
    assert caught > 0

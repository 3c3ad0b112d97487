"""Tree builder against the reference's literal vectors (tree.py:151-245) and
structural properties for every world size."""
import pytest

from tccl_b200 import build_double_tree, build_tree, get_parents_and_children
from tccl_b200.parallel.tree import tree_depths, tree_neighbours


def test_arrays_pow2():
    assert build_double_tree(8) == ([0, 4, 2, 6, 1, 3, 5, 7], [7, 3, 1, 5, 0, 2, 4, 6])
    assert build_double_tree(4) == ([0, 2, 1, 3], [3, 1, 0, 2])
    a, b = build_double_tree(16)
    assert a == [0, 8, 4, 12, 2, 6, 10, 14, 1, 3, 5, 7, 9, 11, 13, 15]
    assert b == [15, 7, 3, 11, 1, 5, 9, 13, 0, 2, 4, 6, 8, 10, 12, 14]
    a, b = build_double_tree(32)
    assert a == [0, 16, 8, 24, 4, 12, 20, 28, 2, 6, 10, 14, 18, 22, 26, 30,
                 1, 3, 5, 7, 9, 11, 13, 15, 17, 19, 21, 23, 25, 27, 29, 31]
    assert b == [31, 15, 7, 23, 3, 11, 19, 27, 1, 5, 9, 13, 17, 21, 25, 29,
                 0, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20, 22, 24, 26, 28, 30]
    assert build_double_tree(2) == ([0, 1], [1, 0])
    assert build_double_tree(1) == ([0], [0])
    assert build_tree(8) == [0, 4, 2, 6, 1, 3, 5, 7]


def test_not_pow2_arrays_rejected():
    with pytest.raises(AssertionError):
        build_tree(6)


def test_neighbours_8():
    exp = [(-1, 4, -1, 1, -1, -1), (2, -1, -1, 3, 0, 2), (4, 1, 3, 1, -1, -1), (2, -1, -1, 7, 1, 5),
           (0, 2, 6, 5, -1, -1), (6, -1, -1, 3, 4, 6), (4, 5, 7, 5, -1, -1), (6, -1, -1, -1, 3, -1)]
    for r in range(8):
        assert get_parents_and_children(8, r) == exp[r]


def test_neighbours_4():
    exp = [(-1, 2, -1, 1, -1, -1), (2, -1, -1, 3, 0, 2), (0, 1, 3, 1, -1, -1), (2, -1, -1, -1, 1, -1)]
    for r in range(4):
        assert get_parents_and_children(4, r) == exp[r]


def test_neighbours_32_samples():
    assert get_parents_and_children(32, 0) == (-1, 16, -1, 1, -1, -1)
    assert get_parents_and_children(32, 7) == (6, -1, -1, 15, 3, 11)
    assert get_parents_and_children(32, 15) == (14, -1, -1, 31, 7, 23)
    assert get_parents_and_children(32, 16) == (0, 8, 24, 17, -1, -1)
    assert get_parents_and_children(32, 23) == (22, -1, -1, 15, 19, 27)
    assert get_parents_and_children(32, 31) == (30, -1, -1, -1, 15, -1)


def test_small_worlds():
    assert get_parents_and_children(1, 0) == (-1, -1, -1, -1, -1, -1)
    assert get_parents_and_children(2, 0) == (-1, 1, -1, 1, -1, -1)
    assert get_parents_and_children(2, 1) == (0, -1, -1, -1, 0, -1)


@pytest.mark.parametrize("N", [2, 4, 8, 16, 32, 64])
def test_heap_arrays_agree_with_neighbours(N):
    for t, arr in enumerate(build_double_tree(N)):
        for i, r in enumerate(arr):
            if i == 0:
                e = (-1, arr[1], -1)
            else:
                e = (arr[i // 2], arr[2 * i] if 2 * i < N else -1, arr[2 * i + 1] if 2 * i + 1 < N else -1)
            assert tree_neighbours(N, r, t) == e


@pytest.mark.parametrize("N", list(range(1, 34)))
def test_any_world_is_two_spanning_trees(N):
    for t in (0, 1):
        roots = 0
        for r in range(N):
            p, l, rr = tree_neighbours(N, r, t)
            roots += p < 0
            for c in (l, rr):
                if c >= 0:
                    assert tree_neighbours(N, c, t)[0] == r
            if p >= 0:
                assert r in tree_neighbours(N, p, t)[1:]
        assert roots == 1
        assert all(d >= 0 for d in tree_depths(N, t))


@pytest.mark.parametrize("N", [2, 4, 8, 16, 32])
def test_leaf_in_one_tree_interior_in_the_other(N):
    for r in range(N):
        a = tree_neighbours(N, r, 0)
        b = tree_neighbours(N, r, 1)
        leaf_a = a[1] < 0 and a[2] < 0
        leaf_b = b[1] < 0 and b[2] < 0
        assert leaf_a != leaf_b

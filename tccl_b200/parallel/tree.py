"""Double binary tree topology (CPU only).

Two complementary binary trees over ``N`` ranks such that every rank is a leaf
in one tree and an interior node (or the single-child "subroot") in the other,
so that a tree all-reduce that sends half of the message over each tree loads
every rank's links equally.  The API and the array form match the reference's
builder (``tree.py:5-148``): ``build_tree`` / ``build_double_tree`` return the
trees in heap order (index 0 = subroot with one child at index 1; the node at
index ``i >= 1`` has its parent at ``i // 2`` and children at ``2 i`` and
``2 i + 1``), and ``get_parents_and_children`` returns
``(a_parent, a_left, a_right, b_parent, b_left, b_right)`` with ``-1`` for
"none".

Unlike the reference (which builds the rows bottom-up and then searches the
list), everything here is closed-form bit arithmetic on the rank:

* tree A: the node at heap index ``i >= 1`` on level ``l = floor(log2 i)`` at
  position ``j = i - 2**l`` is rank ``(2 j + 1) * N / 2**(l + 1)``; a rank's
  level is given by its lowest set bit.
* tree B: tree A with every rank shifted down by one (mod ``N``).

The heap-array form needs a power-of-two ``N``.  The neighbour query is
extended beyond the reference to any ``N >= 1`` (the reference raises for
``N = 1`` and asserts on non powers of two) with the same low-bit rule NCCL
uses for its binary trees, so the kernels can run on 1, 3, 5, 6, 7 GPUs too.
"""
from __future__ import annotations

from functools import lru_cache
from typing import List, Tuple

__all__ = [
    "build_tree",
    "build_double_tree",
    "get_parents_and_children",
    "tree_neighbours",
    "tree_depths",
]


def _is_pow2(n: int) -> bool:
    return n >= 1 and (n & (n - 1)) == 0


def build_tree(N: int) -> List[int]:
    """Tree A in heap order.  ``N`` must be a power of two (``N >= 1``)."""
    if not _is_pow2(N):
        raise AssertionError("len(ranks) is not a power of 2!")
    tree = [0] * N
    for i in range(1, N):
        level = i.bit_length() - 1
        pos = i - (1 << level)
        tree[i] = (2 * pos + 1) * N >> (level + 1)
    return tree


@lru_cache(maxsize=None)
def _double_tree_cached(N: int) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    a = build_tree(N)
    b = [(r - 1) % N for r in a]
    return tuple(a), tuple(b)


def build_double_tree(N: int) -> Tuple[List[int], List[int]]:
    """``(tree_a, tree_b)`` in heap order; ``tree_b[i] = (tree_a[i] - 1) mod N``."""
    a, b = _double_tree_cached(N)
    return list(a), list(b)


def _neighbours_a(N: int, r: int) -> Tuple[int, int, int]:
    """(parent, left, right) of rank ``r`` in tree A for any ``N >= 1``.

    Rank 0 is the subroot: no parent, one child (the root of the in-order
    binary tree over ranks ``1..N-1``).  For ``r >= 1`` with lowest set bit
    ``s``: the children are ``r - s/2`` and ``r + s/2`` (the right child is
    pulled in by halving the step while it falls outside ``N``); the parent is
    whichever of ``r - s`` / ``r + s`` has lowest set bit ``2 s`` and exists,
    else ``r - s``; the top node hangs under the subroot.
    """
    if N == 1:
        return -1, -1, -1
    if r == 0:
        top = 1 << ((N - 1).bit_length() - 1)  # largest power of two <= N-1
        return -1, top, -1
    s = r & -r
    # parent
    up = (r ^ s) | (s << 1)
    if up >= N:
        up = r ^ s
    parent = up  # r ^ s == 0 means "hangs under the subroot", which is rank 0
    # children
    if s == 1:
        return parent, -1, -1
    left = r - (s >> 1)
    step = s >> 1
    right = r + step
    while right >= N and step > 1:
        step >>= 1
        right = r + step
    if right >= N:
        right = -1
    return parent, left, right


def tree_neighbours(N: int, rank: int, tree: int) -> Tuple[int, int, int]:
    """(parent, left, right) of ``rank`` in tree 0 (A) or 1 (B); ``-1`` = none."""
    if not (0 <= rank < N):
        raise ValueError(f"rank {rank} out of range for N={N}")
    if tree == 0:
        return _neighbours_a(N, rank)
    p, l, r = _neighbours_a(N, (rank + 1) % N)
    back = lambda x: -1 if x < 0 else (x - 1) % N
    return back(p), back(l), back(r)


def get_parents_and_children(N: int, rank: int) -> Tuple[int, int, int, int, int, int]:
    """Neighbours of ``rank`` in both trees: A's (parent, left, right) then B's."""
    return (*tree_neighbours(N, rank, 0), *tree_neighbours(N, rank, 1))


def tree_depths(N: int, tree: int) -> List[int]:
    """Depth of every rank below the root of ``tree`` (root = 0)."""
    depth = [-1] * N
    for r in range(N):
        d, x = 0, r
        while True:
            p = tree_neighbours(N, x, tree)[0]
            if p < 0:
                break
            x, d = p, d + 1
            if d > N:
                raise RuntimeError("cycle in tree")
        depth[r] = d
    return depth


def _self_test() -> None:
    """The reference's own check (``tree.py:151-245``): literal trees and neighbour tuples."""
    assert build_double_tree(8) == ([0, 4, 2, 6, 1, 3, 5, 7], [7, 3, 1, 5, 0, 2, 4, 6])
    assert build_double_tree(4) == ([0, 2, 1, 3], [3, 1, 0, 2])
    expect8 = [(-1, 4, -1, 1, -1, -1), (2, -1, -1, 3, 0, 2), (4, 1, 3, 1, -1, -1), (2, -1, -1, 7, 1, 5),
               (0, 2, 6, 5, -1, -1), (6, -1, -1, 3, 4, 6), (4, 5, 7, 5, -1, -1), (6, -1, -1, -1, 3, -1)]
    for r, e in enumerate(expect8):
        assert get_parents_and_children(8, r) == e, (r, get_parents_and_children(8, r))
    a, b = build_double_tree(32)
    assert a[:8] == [0, 16, 8, 24, 4, 12, 20, 28] and b[:8] == [31, 15, 7, 23, 3, 11, 19, 27]
    assert get_parents_and_children(32, 15) == (14, -1, -1, 31, 7, 23)
    for n in range(1, 65):  # any world size: two spanning trees
        for t in (0, 1):
            assert sum(1 for r in range(n) if tree_neighbours(n, r, t)[0] < 0) == 1
            tree_depths(n, t)


if __name__ == "__main__":
    import sys

    _self_test()
    n = int(sys.argv[1]) if len(sys.argv) > 1 else 8
    if _is_pow2(n):
        ta, tb = build_double_tree(n)
        print(f"tree A: {ta}\ntree B: {tb}")
    for r in range(n):
        print(f"rank {r}: {get_parents_and_children(n, r)}")
    print("All passed!")

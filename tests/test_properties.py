"""Property tests (hypothesis) of the host-side decision code: whatever the size, world and settings,
the choices stay inside what the kernels accept."""
import ctypes as C

from hypothesis import given, settings
from hypothesis import strategies as st

from tccl_b200.ops.collectives import _AR_KERNELS, choose_all_reduce_algo
from tccl_b200.ops.fused import ag_pair_schedule
from tccl_b200.ops.tree_allreduce import _tree_grid
from tccl_b200.utils import lib as L
from tccl_b200.utils.consts import K

from test_selection import StubWorld

SLICE_VECS = K["TCCL_TREE_SLICE_BYTES"] // 16


@settings(max_examples=300, deadline=None)
@given(W=st.sampled_from([2, 3, 4, 8]), nvls=st.booleans(), sym=st.booleans(),
       nbytes=st.one_of(st.integers(2, 1 << 12), st.integers(1 << 12, 1 << 22), st.integers(1 << 22, 1 << 31)))
def test_all_reduce_choice_is_always_runnable(W, nvls, sym, nbytes):
    w = StubWorld(W, nvls)
    algo = choose_all_reduce_algo(w, nbytes, sym)
    assert algo in _AR_KERNELS
    if algo.endswith("nvls"):
        assert nvls and W > 2                      # multimem needs the switch; at two ranks it moves more bytes
    if algo.startswith("push"):
        assert nbytes % 16 == 0 and nbytes <= w.push_max_bytes() and nbytes <= w.config.push_max_bytes
    if algo.startswith("twoshot"):
        assert sym                                 # every rank writes its slice into all destinations
    if algo == "twoshot_bulk_p2p":
        assert W == 2 and nbytes >= w.config.bulk_min_bytes


@settings(max_examples=300, deadline=None)
@given(W=st.sampled_from([1, 2, 3, 4, 5, 8]), sms=st.sampled_from([16, 64, 132, 148]),
       vecs=st.integers(1, 1 << 26), ctas=st.integers(1, 128),
       chunk=st.sampled_from([1024, 4096, 65536, 1 << 20, 4 << 20, 16 << 20, 64 << 20]))
def test_tree_grid_always_fits_the_ring(W, sms, vecs, ctas, chunk):
    w = StubWorld(W, True, sms=sms, tree_ctas=ctas, tree_chunk_bytes=chunk)
    k, chunk_vecs = _tree_grid(w, vecs * 16)
    assert 1 <= k <= min(ctas, K["TCCL_TREE_MAX_CTAS"], max(1, w.max_ctas() // 4))
    assert 1 <= chunk_vecs <= k * SLICE_VECS       # a CTA moves at most one ring slice of a chunk


@settings(max_examples=60, deadline=None)
@given(W=st.sampled_from([2, 3, 4, 8]), tm2=st.integers(1, 4), tn=st.integers(1, 9), pairs=st.integers(1, 74),
       nbatch=st.integers(1, 8), ring=st.booleans(), halves=st.booleans(), k=st.sampled_from([64, 1024, 8192]),
       tflops=st.floats(1.0, 40.0), gbs=st.floats(50.0, 900.0))
def test_ag_plan_covers_every_tile_once_for_any_cost_model(W, tm2, tn, pairs, nbatch, ring, halves, k, tflops, gbs):
    tm = 2 * tm2
    rank = (W * 7 + tn) % W
    plan = ag_pair_schedule(W, rank, tm, tn, pairs, min(nbatch, tm), k, halves=halves, ring=ring,
                            pair_tflops=tflops, link_gbs=gbs)
    seen = {}
    for units in plan:
        for mt, nt, half in units:
            assert mt % 2 == 0 and 0 <= mt < W * tm and 0 <= nt < tn and half in (0, 1, 2)
            assert mt < (1 << 12) and nt < (1 << 16)   # the fields of a packed table entry
            seen.setdefault((mt, nt), []).append(half)
    assert len(plan) == pairs and len(seen) == W * tm2 * tn
    assert all(v == [0] or sorted(v) == [1, 2] for v in seen.values())


def test_bulk_copy_stages_fit_shared_memory_for_every_world():
    lib = L.lib()
    lib.tccl_allreduce_bulk_chunk_bytes.restype = C.c_uint32
    for W in range(1, K["TCCL_MAX_WORLD"] + 1):
        chunk = int(lib.tccl_allreduce_bulk_chunk_bytes(W))
        assert chunk >= 4096 and chunk % 1024 == 0 and chunk <= 16384
        assert (3 * W + 2) * chunk <= 192 * 1024   # three input stages of W chunks + two output stages

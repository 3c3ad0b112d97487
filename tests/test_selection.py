"""Host-side decision logic that needs no GPU: kernel choice by message size and world,
grid sizing, tree chunking, weight packing."""
import pytest
import torch

from tccl_b200.config import Config
from tccl_b200.ops._common import grid_for
from tccl_b200.ops.collectives import choose_all_reduce_algo
from tccl_b200.ops.fused import pack_gate_up
from tccl_b200.ops.tree_allreduce import _tree_grid
from tccl_b200.parallel.world import PlanCache, WorldBase
from tccl_b200.utils.consts import K


class StubWorld(WorldBase):
    """The few attributes the selection code reads from a communicator."""

    def __init__(self, world_size, nvls, sms=148, **cfg):
        self.world_size, self._nvls, self._sms = world_size, nvls, sms
        self.config = Config()
        for k, v in cfg.items():
            setattr(self.config, k, v)
        self.ll_bytes = 2 << 20

    has_nvls = property(lambda self: self._nvls)

    def num_sms(self):
        return self._sms

    def max_ctas(self):
        return max(1, min(self.config.max_ctas or self._sms, K["TCCL_MAX_BLOCKS"]))

    def local_copy_ctas(self):
        return min(4 * self.max_ctas(), K["TCCL_MAX_BLOCKS"])


def test_all_reduce_choice_follows_size_and_world():
    w8 = StubWorld(8, True)
    assert choose_all_reduce_algo(w8, 4096, True) == "push_nvls"
    assert choose_all_reduce_algo(w8, 64 * 1024, False) == "push_nvls"
    assert choose_all_reduce_algo(w8, 64 * 1024, True) == "twoshot_nvls"      # a switch and a symmetric destination
    assert choose_all_reduce_algo(w8, 256 * 1024, True) == "twoshot_nvls"
    assert choose_all_reduce_algo(w8, 256 * 1024, False) == "oneshot_nvls"
    assert choose_all_reduce_algo(w8, 16 << 20, True) == "twoshot_nvls"
    assert choose_all_reduce_algo(w8, 16 << 20, False).startswith("oneshot")  # no symmetric destination
    assert choose_all_reduce_algo(w8, 4100, True) == "oneshot_nvls"           # not a multiple of 16 bytes: no push
    w2 = StubWorld(2, True)  # two ranks: NVLS moves more bytes than P2P
    assert choose_all_reduce_algo(w2, 4096, True) == "push_p2p"
    assert choose_all_reduce_algo(w2, 32 << 20, True) == "twoshot_p2p"
    assert choose_all_reduce_algo(w2, 64 << 20, True) == "twoshot_bulk_p2p"  # two ranks, large: bulk copies
    w4 = StubWorld(4, False)
    assert choose_all_reduce_algo(w4, 64 << 20, True) == "twoshot_p2p"
    assert choose_all_reduce_algo(StubWorld(1, False), 1 << 30, True) == "oneshot_p2p"
    forced = StubWorld(8, True, force_variant="twoshot_p2p")
    assert choose_all_reduce_algo(forced, 8, True) == "twoshot_p2p"


def test_grid_is_a_function_of_size_and_shared_config_only():
    w = StubWorld(8, True)
    assert grid_for(w, 1, 512, 4) == 1
    assert grid_for(w, 512 * 4 * 3 + 1, 512, 4) == 4
    assert grid_for(w, 1 << 30, 512, 4) == 148
    assert grid_for(w, 1 << 30, 512, 8, cap=8) == 8
    assert grid_for(StubWorld(8, True, max_ctas=32), 1 << 30, 512, 4) == 32
    assert grid_for(StubWorld(1, False), 1 << 30, 512, 8) == 592  # one rank: a local copy, several CTAs per SM


def test_tree_grid_fits_the_ring_and_scales_ctas_with_the_message():
    w = StubWorld(8, True)
    slice_vecs = K["TCCL_TREE_SLICE_BYTES"] // 16
    k, vecs = _tree_grid(w, 1 << 30)
    assert k == w.config.tree_ctas == 36 and vecs == k * slice_vecs  # large: every CTA moves a full ring slice per chunk
    k, vecs = _tree_grid(w, 1 << 20)
    assert k == 16 and vecs <= k * slice_vecs and (1 << 20) // 2 // (vecs * 16) >= 4  # >= 4 chunks per tree
    k, vecs = _tree_grid(w, 4096)
    assert k == 1 and vecs >= 1                        # small: one CTA per role
    small = StubWorld(8, True, tree_chunk_bytes=1024)
    k, vecs = _tree_grid(small, 1 << 20)
    assert vecs == 64 and vecs <= k * slice_vecs       # small chunks on request


def test_pack_gate_up_layout():
    F, Kd = 256, 8
    gate = torch.arange(F * Kd, dtype=torch.float32).view(F, Kd)
    up = -gate
    p = pack_gate_up(gate, up)
    assert p.shape == (2 * F, Kd)
    assert torch.equal(p[:128], gate[:128]) and torch.equal(p[128:256], up[:128])
    assert torch.equal(p[256:384], gate[128:]) and torch.equal(p[384:], up[128:])


def test_plan_cache_is_bounded_and_evicts_the_least_recently_used():
    c = PlanCache(3)
    for k in "abc":
        c.insert(k, k.upper())
    assert c.lookup("a") == "A"          # refreshes "a"
    c.insert("d", "D")                   # evicts "b", the least recently used
    assert c.lookup("b") is None and len(c) == 3
    assert [c.lookup(k) for k in "acd"] == ["A", "C", "D"]
    c.clear()
    assert len(c) == 0


def test_plan_key_tells_a_strided_view_from_a_contiguous_tensor():
    from tccl_b200.ops.collectives import _tkey

    base = torch.zeros(64)
    a, b = base[:16], base[:32:2]       # same address, element count and dtype; different layout
    assert a.data_ptr() == b.data_ptr() and a.numel() == b.numel()
    assert _tkey(a) != _tkey(b)
    assert _tkey(a) == _tkey(base[:16])


def test_push_slot_is_fixed_per_world_not_per_message():
    w8, w3 = StubWorld(8, True), StubWorld(3, False)
    assert w8.push_max_bytes() == (2 << 20) // 16
    assert w3.push_max_bytes() % 16 == 0 and 2 * 3 * w3.push_max_bytes() <= w3.ll_bytes


@pytest.mark.parametrize("W,tm,tn,pairs,nbatch", [(8, 4, 7, 74, 2), (8, 4, 7, 74, 4), (4, 8, 14, 74, 2), (2, 16, 28, 74, 2),
                                                  (2, 2, 1, 4, 1), (3, 2, 3, 5, 2), (8, 2, 2, 74, 3)])
def test_ag_pair_schedule_names_every_tile_once(W, tm, tn, pairs, nbatch):
    """Whatever the cost model says, a plan must hold every tile exactly once: whole, or as its two halves."""
    from tccl_b200.ops.fused import ag_pair_schedule

    for rank in range(W):
        for halves, ring in ((True, False), (False, False), (True, True), (False, True)):
            plan = ag_pair_schedule(W, rank, tm, tn, pairs, nbatch, 512, halves=halves, ring=ring)
            assert len(plan) == pairs
            seen = {}
            for units in plan:
                for mt, nt, half in units:
                    assert mt % 2 == 0 and 0 <= mt < W * tm and 0 <= nt < tn and half in (0, 1, 2)
                    seen.setdefault((mt, nt), []).append(half)
            assert len(seen) == W * (tm // 2) * tn
            assert all(v == [0] or sorted(v) == [1, 2] for v in seen.values())
            if not halves:
                assert all(v == [0] for v in seen.values())
            # the rank's own rows need no data from anybody: they come first wherever a pair has one
            for units in plan:
                own = [i for i, (mt, _, _) in enumerate(units) if mt // tm == rank]
                assert own == list(range(len(own))) or W == 1

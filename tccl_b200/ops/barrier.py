"""Device barriers between the ranks of a world.

``barrier`` runs the library's epoch barrier (posted release stores + acquire
polls on the library's own flag region; ``flavour="nvls"`` signals all peers
with one ``multimem.red``).  ``barrier_test`` is the counterpart of the
reference's ``barrier_test(symm_mem)`` (``triton_barrier.py:154-159``): the
self-resetting CAS protocol on the *signal pads of a torch symmetric-memory
handle*, ``[block][world]`` layout, pads all zero again afterwards.
"""
from __future__ import annotations

from typing import Optional

from ..parallel.world import WorldBase
from ..utils import lib as L
from ._common import K, get_world

__all__ = ["barrier", "barrier_test", "wait_never"]


def barrier(world: Optional[WorldBase] = None, *, blocks: int = 1, threads: int = 32, rounds: int = 1,
            flavour: str = "p2p") -> None:
    w = get_world(world)
    if not (1 <= blocks <= K["TCCL_MAX_BLOCKS"]):
        raise ValueError("blocks out of range")
    if flavour == "nvls" and not w.has_nvls:
        raise RuntimeError("nvls barrier needs NVLS multicast")
    args = {r: L.BarrierArgs(rounds) for r in w.local_ranks}
    w.launch("tccl_barrier_nvls" if flavour == "nvls" else "tccl_barrier_p2p", args, blocks, max(threads, 32))


def barrier_test(symm_mem=None, world: Optional[WorldBase] = None, *, blocks: int = 32, threads: int = 128,
                 pads=None) -> None:
    """CAS barrier on signal pads.  Real world: pass the torch symmetric-memory
    handle (``rendezvous`` result).  Emulated world: pass ``pads`` = an
    ``EmuTensor`` of uint32/int32 pads."""
    w = get_world(world)
    W = w.world_size
    a = L.PadsArgs()
    if symm_mem is not None:
        ptrs = [int(p) for p in symm_mem.signal_pad_ptrs]
        size = int(getattr(symm_mem, "signal_pad_size", blocks * W * 4))
    else:
        ptrs = w.peer_ptrs(pads)
        size = pads.numel() * 4
    if blocks * W * 4 > size:
        raise ValueError(f"signal pad too small for {blocks} blocks x {W} ranks")
    for p, v in enumerate(ptrs):
        a.pads[p] = v
    w.launch("tccl_barrier_cas", {r: a for r in w.local_ranks}, blocks, max(threads, 32))


def wait_never(world: Optional[WorldBase] = None) -> None:
    """Launch a kernel whose wait can never be satisfied (nothing sets the flag);
    it returns after the configured timeout with a TIMEOUT status.  Test hook for
    the failure-reporting path — it does not hang or fault the GPU."""
    w = get_world(world)
    w.launch("tccl_wait_never", {r: L.BarrierArgs(0) for r in w.local_ranks}, 1, 32)

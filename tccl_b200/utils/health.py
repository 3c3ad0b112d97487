"""Host-side failure detection between steps.

The device kernels bound every wait, so a dead peer costs one timeout and an
error status rather than a hang — but the cheap way to learn that a rank is
gone is on the host, *before* the next kernel is launched.  ``PeerMonitor``
keeps one heartbeat counter per rank in the process group's key-value store:
every rank bumps its own counter once per step (``beat``) and looks at the
others' (``check``); a rank whose counter has not moved for ``stale_s`` seconds,
or that announced its departure with ``leave``, is reported as lost and the
caller can stop launching, shrink the group or re-rendezvous.  A rank may only
leave between steps, with none of its kernels or collectives in flight.

The reference has no failure handling of any kind (unbounded spins, no
timeouts: ``triton_barrier.py:108-118``).
"""
from __future__ import annotations

import time
from typing import Dict, List


class PeerLost(RuntimeError):
    def __init__(self, ranks: List[int], why: Dict[int, str]):
        super().__init__(f"lost ranks {ranks}: {why}")
        self.ranks, self.why = ranks, why


class PeerMonitor:
    def __init__(self, store, rank: int, world_size: int, stale_s: float = 5.0, prefix: str = "tccl/hb"):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.stale_s, self.prefix = stale_s, prefix
        self._seen: Dict[int, tuple] = {}  # rank -> (counter, time it last changed)
        self._step = 0
        self.store.set(self._key(rank), "0")

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        """Call once per step, before launching it."""
        self._step += 1
        self.store.set(self._key(self.rank), str(self._step))

    def leave(self) -> None:
        """Announce an orderly departure (between steps only)."""
        self.store.set(self._key(self.rank), "left")

    def lost(self) -> Dict[int, str]:
        now = time.monotonic()
        bad: Dict[int, str] = {}
        for r in range(self.world_size):
            if r == self.rank:
                continue
            try:
                if not self.store.check([self._key(r)]):
                    val = None
                else:
                    val = self.store.get(self._key(r)).decode()
            except Exception as e:  # noqa: BLE001 - a store error is itself a lost-peer signal
                bad[r] = f"store error: {type(e).__name__}"
                continue
            if val == "left":
                bad[r] = "left"
                continue
            prev = self._seen.get(r)
            if prev is None or prev[0] != val:
                self._seen[r] = (val, now)
            elif now - prev[1] > self.stale_s:
                bad[r] = f"no heartbeat for {now - prev[1]:.1f} s"
        return bad

    def check(self) -> None:
        """Raise ``PeerLost`` if a peer left or went silent."""
        bad = self.lost()
        if bad:
            raise PeerLost(sorted(bad), bad)

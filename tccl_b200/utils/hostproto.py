"""CPU ranks running the device protocols' host twin (csrc/host/host_protocol.cpp)
over POSIX shared memory.  Used by the failure-handling tests: faults are
injected here, never on a GPU."""
from __future__ import annotations

import ctypes as C
import multiprocessing as mp
from multiprocessing import shared_memory
from typing import Dict, List, Optional

import numpy as np

from ..parallel.tree import tree_neighbours
from .consts import K, MAX_WORLD as MAXW


class HpComm(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("flags", C.c_uint64 * MAXW), ("local", C.c_uint64),
                ("timeout_ns", C.c_uint64)]


class HpFaults(C.Structure):
    _fields_ = [("drop_signal_to", C.c_int32), ("stall_ms", C.c_int32), ("stop_after_chunk", C.c_int32)]


class HpTree(C.Structure):
    _fields_ = [("inp", C.c_uint64), ("buf", C.c_uint64 * MAXW), ("ring", C.c_uint64 * MAXW),
                ("numel", C.c_uint64), ("chunk", C.c_uint64), ("ring_stride", C.c_uint64),
                ("parent", C.c_int32 * 2), ("left", C.c_int32 * 2), ("right", C.c_int32 * 2),
                ("child_slot", C.c_int32 * 2), ("pull_down", C.c_int32), ("pad_", C.c_int32)]


def _lib(path: Optional[str] = None) -> C.CDLL:
    if path is None:
        from . import build as B

        path = B.build_host()
    lib = C.CDLL(str(path))
    lib.hp_barrier.restype = C.c_int
    lib.hp_tree_allreduce.restype = C.c_int
    return lib


def layout(world: int, numel: int):
    """Byte offsets inside the shared block: flag regions, private words, data buffers, and the
    double-tree rings (sized for chunks of up to ``numel`` elements)."""
    fb, lb, db = K["TCCL_FLAG_WORDS"] * 4, K["TCCL_LOCAL_WORDS"] * 4, numel * 4
    rb = 4 * K["TCCL_TREE_RING_DEPTH"] * db
    flags = [r * fb for r in range(world)]
    local = [world * fb + r * lb for r in range(world)]
    data = [world * (fb + lb) + r * db for r in range(world)]
    rings = [world * (fb + lb + db) + r * rb for r in range(world)]
    return flags, local, data, rings, world * (fb + lb + db + rb)


def _status(buf, off) -> dict:
    w = np.frombuffer(buf, dtype=np.uint32, count=K["TCCL_ST_WORDS"], offset=off + K["TCCL_LOCAL_STATUS"] * 4)
    names = {v: k for k, v in K.items() if k.startswith("TCCL_W_")}
    peer = int(w[K["TCCL_ST_PEER"]])
    return {"code": int(w[K["TCCL_ST_CODE"]]), "block": int(w[K["TCCL_ST_BLOCK"]]),
            "peer": -1 if peer == 0xFFFFFFFF else peer, "where": names.get(int(w[K["TCCL_ST_WHERE"]]), "?"),
            "aborted": bool(w[K["TCCL_ST_ABORT"]])}


def _rank_main(lib_path: str, shm_name: str, world: int, rank: int, numel: int, op: str, timeout_ms: float,
               faults: dict, q):
    shm = shared_memory.SharedMemory(name=shm_name)
    try:
        base = C.addressof(C.c_char.from_buffer(shm.buf))
        flags, local, data, rings, _ = layout(world, numel)
        lib = _lib(lib_path)
        comm = HpComm()
        comm.world, comm.rank = world, rank
        for p in range(world):
            comm.flags[p] = base + flags[p]
        comm.local = base + local[rank]
        comm.timeout_ns = int(timeout_ms * 1e6)
        f = HpFaults(faults.get("drop_signal_to", -1), faults.get("stall_ms", 0), faults.get("stop_after_chunk", -1))
        if faults.get("never_join"):
            q.put((rank, None, None))
            return
        if op == "barrier":
            ok = lib.hp_barrier(C.byref(comm), 0, int(faults.get("rounds", 1)), C.byref(f))
        else:
            t = HpTree()
            t.inp = base + data[rank]  # in place: the result buffer is the input
            for p in range(world):
                t.buf[p] = base + data[p]
                t.ring[p] = base + rings[p]
            t.numel, t.chunk = numel, int(faults.get("chunk", max(1, numel // 16)))
            t.ring_stride = numel
            t.pull_down = int(faults.get("pull_down", 0))
            for tr in (0, 1):
                parent, left, right = tree_neighbours(world, rank, tr)
                t.parent[tr], t.left[tr], t.right[tr] = parent, left, right
                t.child_slot[tr] = 0 if parent < 0 or tree_neighbours(world, parent, tr)[1] == rank else 1
            ok = lib.hp_tree_allreduce(C.byref(comm), C.byref(t), C.byref(f))
        q.put((rank, int(ok), _status(shm.buf, local[rank])))
    finally:
        del base
        shm.close()


def run_ranks(world: int, op: str, numel: int = 0, inputs: Optional[List[np.ndarray]] = None, timeout_ms: float = 2000.0,
              faults: Optional[Dict[int, dict]] = None, join_s: float = 30.0):
    """Run ``op`` ("barrier" or "tree") on ``world`` CPU processes.  ``faults`` maps a
    rank to its injected fault.  Returns (results by rank, output arrays or None)."""
    from . import build as B

    lib_path = str(B.build_host())  # built once here; the ranks only load it
    faults = faults or {}
    flags, local, data, rings, total = layout(world, numel)
    shm = shared_memory.SharedMemory(create=True, size=max(total, 4096))
    try:
        np.frombuffer(shm.buf, dtype=np.uint8)[:] = 0
        if inputs is not None:
            for r in range(world):
                np.frombuffer(shm.buf, dtype=np.float32, count=numel, offset=data[r])[:] = inputs[r]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_rank_main, args=(lib_path, shm.name, world, r, numel, op, timeout_ms, faults.get(r, {}), q))
                 for r in range(world)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(world):
            rank, ok, st = q.get(timeout=join_s)
            results[rank] = {"ok": ok, "status": st}
        for p in procs:
            p.join(timeout=join_s)
        outs = None
        if inputs is not None:
            outs = [np.frombuffer(shm.buf, dtype=np.float32, count=numel, offset=data[r]).copy() for r in range(world)]
        return results, outs
    finally:
        shm.close()
        shm.unlink()

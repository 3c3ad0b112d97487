"""Communicator objects.

``RealWorld`` is one rank of a ``torch.distributed`` process group whose
tensors live in PyTorch symmetric memory (``torch.distributed._symmetric_memory``:
``empty`` + ``rendezvous`` give the peer-mapped buffer pointers and, on
NVSwitch systems, the multicast alias).  ``EmuWorld`` (``parallel/emu.py``) runs
all ranks of a small world on ONE GPU inside one cooperative launch, which is
how the multi-rank protocols are tested where only one GPU is present.

Both expose the same small interface to the ops layer:

* ``local_ranks`` — ranks this process drives (one, or all W when emulated)
* ``peer_ptrs(x)`` / ``mc_ptr(x)`` — device addresses of every rank's copy of
  the symmetric tensor ``x`` (view offset applied) and of its multicast alias
* ``local(x, r)`` — rank ``r``'s own ``torch.Tensor``
* ``launch(name, args_by_rank, grid, block, dtype)`` — one kernel launch

The reference does the equivalent bring-up inline in every script
(``triton_barrier.py:162-181``) and re-runs ``rendezvous`` on every call
(``triton_one_shot_all_reduce_no_128.py:82``); here the handle of an allocation
is resolved once and cached.
"""
from __future__ import annotations

import ctypes as C
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence

import torch

from ..config import Config
from ..utils import lib as L

K = L.K


def _status_dict(words: Sequence[int]) -> dict:
    where_names = {v: k for k, v in K.items() if k.startswith("TCCL_W_")}
    return {
        "code": int(words[K["TCCL_ST_CODE"]]),
        "block": int(words[K["TCCL_ST_BLOCK"]]),
        "peer": int(words[K["TCCL_ST_PEER"]]) if words[K["TCCL_ST_PEER"]] != 0xFFFFFFFF else -1,
        "where": where_names.get(int(words[K["TCCL_ST_WHERE"]]), str(int(words[K["TCCL_ST_WHERE"]]))),
        "seen": int(words[K["TCCL_ST_SEEN"]]),
        "want": int(words[K["TCCL_ST_WANT"]]),
        "aborted": bool(words[K["TCCL_ST_ABORT"]]),
    }


class PlanCache(OrderedDict):
    """Least-recently-used cache of plans (``Config.plan_cache_size`` entries)."""

    def __init__(self, maxsize: int = 512):
        super().__init__()
        self.maxsize = max(1, int(maxsize))

    def lookup(self, key):
        p = self.get(key)
        if p is not None:
            self.move_to_end(key)
        return p

    def insert(self, key, plan):
        self[key] = plan
        while len(self) > self.maxsize:
            self.popitem(last=False)


def tree_ring_bytes(config: Config) -> int:
    """Bytes of the double-tree ring: the small-message part, then [tree][child slot][cta][depth] slices
    for ``tree_ctas`` CTAs per role."""
    k = max(1, min(int(config.tree_ctas), K["TCCL_TREE_MAX_CTAS"]))
    return K["TCCL_TREE_LL_BYTES"] + 4 * k * K["TCCL_TREE_RING_DEPTH"] * K["TCCL_TREE_SLICE_BYTES"]


class WorldBase:
    """What the ops layer needs from a communicator."""

    world_size: int
    config: Config
    device: torch.device
    launches: int = 0  # kernels of this library launched so far

    # -- to be provided by subclasses
    @property
    def local_ranks(self) -> List[int]:
        raise NotImplementedError

    @property
    def has_nvls(self) -> bool:
        raise NotImplementedError

    def peer_ptrs(self, x) -> List[int]:
        raise NotImplementedError

    def mc_ptr(self, x) -> int:
        raise NotImplementedError

    def local(self, x, r: int) -> torch.Tensor:
        raise NotImplementedError

    def wrap(self, per_rank: Dict[int, torch.Tensor]):
        """Turn {rank: tensor} into what this world hands back to the user."""
        raise NotImplementedError

    def prepare(self, name: str, args_by_rank: Dict[int, C.Structure], grid: int, block: int,
                dtype_code: int = 0):
        """Bind one kernel launch to its arguments; returns a zero-argument callable
        that enqueues it on the current stream.  The argument structs stay owned by
        the caller, who may patch a field (an output pointer) between calls."""
        raise NotImplementedError

    def launch(self, name: str, args_by_rank: Dict[int, C.Structure], grid: int, block: int,
               dtype_code: int = 0) -> None:
        self.prepare(name, args_by_rank, grid, block, dtype_code)()

    def empty(self, shape, dtype=torch.bfloat16):
        raise NotImplementedError

    # -- shared helpers
    def num_sms(self) -> int:
        if not hasattr(self, "_sms"):
            self._sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        return self._sms

    def max_ctas(self) -> int:
        m = self.config.max_ctas or self.num_sms()
        return max(1, min(m, K["TCCL_MAX_BLOCKS"]))

    def local_copy_ctas(self) -> int:
        """A one-rank collective is a local copy: HBM-bound, wants several CTAs per SM."""
        return min(4 * self.max_ctas(), K["TCCL_MAX_BLOCKS"])

    def push_max_bytes(self) -> int:
        """Largest message of the push all-reduce: one slot of the small-message region
        (two alternating halves of ``world_size`` fixed slots each)."""
        return (self.ll_bytes // 2 // self.world_size) & ~15

    def coll_flags(self, sync_entry: bool = True, sync_exit: bool = True) -> int:
        f = 0
        if not sync_entry:
            f |= K["TCCL_F_NO_ENTRY_BARRIER"]
        if not sync_exit:
            f |= K["TCCL_F_NO_EXIT_BARRIER"]
        if self.config.nvls_barrier and self.has_nvls:
            f |= K["TCCL_F_NVLS_BARRIER"]
        return f


class RealWorld(WorldBase):
    """One rank of a process group over PyTorch symmetric memory."""

    def __init__(self, group=None, config: Optional[Config] = None, device=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        if not dist.is_initialized():
            raise RuntimeError("call torch.distributed.init_process_group first")
        if not torch.cuda.is_available():
            raise RuntimeError("tccl_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        self._dist, self._symm = dist, symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.config = config or Config.from_env()
        self.world_size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world_size > L.MAX_WORLD:
            raise ValueError(f"world size {self.world_size} > {L.MAX_WORLD}")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        L.lib()  # fail loudly if the native library is absent
        try:  # still needed by older symmetric-memory builds; newer ones only warn that it is deprecated
            import warnings

            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except (AttributeError, TypeError):  # the function is gone or changed its signature: nothing to enable
            pass
        self._handles: Dict[int, tuple] = {}
        self.plans = PlanCache(self.config.plan_cache_size)  # op wrappers cache their bound launches here
        # workspace = [flag region | staging area], one symmetric allocation
        self._flag_bytes = -(-K["TCCL_FLAG_WORDS"] * 4 // 65536) * 65536
        self._stage_bytes = int(self.config.stage_mb) << 20
        self.tree_bytes = tree_ring_bytes(self.config)
        self.workspace = symm_mem.empty(self._flag_bytes + self._stage_bytes + self.tree_bytes, dtype=torch.uint8,
                                        device=self.device)
        self.workspace[: self._flag_bytes].zero_()
        self._zero_tree_ll()
        self.local_state = torch.zeros(K["TCCL_LOCAL_WORDS"], dtype=torch.int32, device=self.device)
        ptrs, mc = self._resolve(self.workspace)
        self._nvls = bool(mc) and not self.config.disable_nvls
        comm = L.Comm()
        comm.world, comm.rank = self.world_size, self.rank
        for p in range(self.world_size):
            comm.flags[p] = ptrs[p]
            comm.stage[p] = ptrs[p] + self._flag_bytes
        comm.mc_flags = mc if mc else 0
        comm.mc_stage = (mc + self._flag_bytes) if mc else 0
        comm.local = self.local_state.data_ptr()
        # the tail of the staging area belongs to the small-message push all-reduce (it runs
        # without an entry barrier, so it must not share slots with the fused GEMM kernels)
        self.ll_bytes = min(2 << 20, self._stage_bytes // 4)
        comm.stage_bytes = self._stage_bytes - self.ll_bytes
        comm.timeout_ns = self.config.timeout_ns
        comm.ll_bytes = self.ll_bytes
        comm.tree_bytes = self.tree_bytes  # the double-tree ring follows the staging area
        self.comm = comm
        self._stage_ptrs = [ptrs[p] + self._flag_bytes for p in range(self.world_size)]
        self._stage_mc = (mc + self._flag_bytes) if mc else 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # -- symmetric tensors
    def empty(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """Allocate a tensor in symmetric memory (collective: every rank calls
        it with the same shape) and resolve its peer pointers once."""
        if isinstance(shape, int):
            shape = (shape,)
        t = self._symm.empty(*shape, dtype=dtype, device=self.device)
        self._resolve(t)
        return t

    def _resolve(self, t: torch.Tensor):
        key = t.untyped_storage().data_ptr()
        ent = self._handles.get(key)
        if ent is None:
            hdl = self._symm.rendezvous(t, self.group)
            if hdl is None:
                raise ValueError("this tensor does not live in symmetric memory: allocate it with "
                                 "tccl_b200.empty() / world.empty() (or torch.distributed._symmetric_memory.empty)")
            base = [int(p) for p in hdl.buffer_ptrs]
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            # the entry keeps `t` alive: a symmetric allocation stays mapped (and its
            # address cannot be reused by another allocation) until free() drops it
            ent = (hdl, base, mc, base[self.rank], t)
            self._handles[key] = ent
        hdl, base, mc, local_base = ent[:4]
        delta = t.data_ptr() - local_base
        return [b + delta for b in base], (mc + delta if mc else 0)

    def _zero_tree_ll(self) -> None:
        """The small-message tree slots are read before they are ever written (flags travel inside the
        data): they must not start out with bits that look like a flag."""
        lo = self._flag_bytes + self._stage_bytes
        self.workspace[lo: lo + K["TCCL_TREE_LL_BYTES"]].zero_()

    def free(self, t: torch.Tensor) -> None:
        """Forget a symmetric allocation (and every cached launch that points into it)."""
        self._handles.pop(t.untyped_storage().data_ptr(), None)
        self.plans.clear()

    def handle(self, t: torch.Tensor):
        """The torch symmetric-memory handle of ``t``'s allocation."""
        self._resolve(t)
        return self._handles[t.untyped_storage().data_ptr()][0]

    # -- WorldBase interface
    @property
    def local_ranks(self) -> List[int]:
        return [self.rank]

    @property
    def has_nvls(self) -> bool:
        return self._nvls

    def peer_ptrs(self, x: torch.Tensor) -> List[int]:
        return self._resolve(x)[0]

    def mc_ptr(self, x: torch.Tensor) -> int:
        return self._resolve(x)[1] if self._nvls else 0

    def local(self, x: torch.Tensor, r: int) -> torch.Tensor:
        return x

    def wrap(self, per_rank):
        return per_rank[self.rank]

    def stage_ptrs(self) -> List[int]:
        return self._stage_ptrs

    def stage_mc(self) -> int:
        return self._stage_mc if self._nvls else 0

    def ll_ptrs(self) -> List[int]:
        off = self._stage_bytes - self.ll_bytes
        return [p + off for p in self._stage_ptrs]

    def ll_mc(self) -> int:
        return (self._stage_mc + self._stage_bytes - self.ll_bytes) if self._nvls and self._stage_mc else 0

    def stage_view(self, nbytes: int, dtype=torch.uint8, offset: int = 0) -> torch.Tensor:
        """A local tensor view of this rank's staging area."""
        if offset + nbytes > self._stage_bytes:
            raise ValueError(f"staging area too small: need {offset + nbytes}, have {self._stage_bytes}")
        raw = self.workspace[self._flag_bytes + offset : self._flag_bytes + offset + nbytes]
        return raw.view(dtype)

    def prepare(self, name, args_by_rank, grid, block, dtype_code=0):
        fn = getattr(L.lib(), name)
        a = args_by_rank[self.rank]
        l = L.Launch(int(grid), int(block), 0, int(dtype_code), None)
        comm_ref, a_ref, l_ref = C.byref(self.comm), C.byref(a), C.byref(l)
        raw_stream = torch._C._cuda_getCurrentRawStream
        dev = self.device.index

        def go():
            l.stream = raw_stream(dev)
            rc = fn(comm_ref, a_ref, l_ref)
            if rc:
                L.check(rc, name)
            self.launches += 1

        go.keep = (a, l)  # the structs the references point into
        return go

    # -- state
    def last_status(self) -> dict:
        w = self.local_state[K["TCCL_LOCAL_STATUS"] : K["TCCL_LOCAL_STATUS"] + K["TCCL_ST_WORDS"]].cpu().tolist()
        return _status_dict([x & 0xFFFFFFFF for x in w])

    def check(self) -> None:
        """Synchronise and raise ``TcclTimeout`` if a device wait gave up."""
        st = self.last_status()
        if st["code"] != 0:
            raise L.TcclTimeout(st)

    def reset(self) -> None:
        """Collective: bring flags, epochs and status back to zero on all ranks."""
        torch.cuda.synchronize(self.device)
        self._dist.barrier(self.group)
        self.workspace[: self._flag_bytes].zero_()
        self._zero_tree_ll()
        self.local_state.zero_()
        for k in ("_ag_seq", "_stage_user"):  # host-side mirrors of device state
            self.__dict__.pop(k, None)
        torch.cuda.synchronize(self.device)
        self._dist.barrier(self.group)

    def set_timeout_ms(self, ms: float) -> None:
        self.config.timeout_ms = ms
        self.comm.timeout_ns = self.config.timeout_ns

    def reconfigure(self, **kw) -> None:
        """Change configuration fields (identically on every rank) and drop the
        cached launches that were sized with the old values."""
        for k, v in kw.items():
            if not hasattr(self.config, k):
                raise AttributeError(k)
            setattr(self.config, k, v)
        self.comm.timeout_ns = self.config.timeout_ns
        self.plans.clear()

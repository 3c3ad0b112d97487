"""All ranks of a small world on one GPU.

Kernels that wait on one another must never run as separate launches on one
GPU (nothing guarantees they run at the same time), so an emulated world runs
every collective as ONE cooperative launch whose ``blockIdx.y`` is the rank;
the W "peer" buffers are ordinary allocations on the same device.  All P2P
protocols (barriers, flat collectives, the double tree, the fused GEMM ops)
run unchanged; only the NVLS variants need real multicast hardware.

A symmetric tensor is an ``EmuTensor``: a list-like of W per-rank tensors.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..config import Config
from ..utils import lib as L
from .world import WorldBase, _status_dict, tree_ring_bytes

K = L.K


class EmuTensor:
    """W same-shaped tensors on one device standing in for one symmetric tensor."""

    def __init__(self, parts: List[torch.Tensor]):
        self.parts = parts

    def __getitem__(self, r):
        if isinstance(r, int):
            return self.parts[r]
        return EmuTensor([p[r] for p in self.parts])  # a view of every rank's copy

    def __len__(self):
        return len(self.parts)

    def __iter__(self):
        return iter(self.parts)

    @property
    def shape(self):
        return self.parts[0].shape

    @property
    def dtype(self):
        return self.parts[0].dtype

    def numel(self):
        return self.parts[0].numel()

    def view_all(self, fn) -> "EmuTensor":
        return EmuTensor([fn(p) for p in self.parts])


class EmuWorld(WorldBase):
    def __init__(self, world_size: int, config: Optional[Config] = None, device="cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("EmuWorld needs a CUDA device")
        if not (1 <= world_size <= L.MAX_WORLD):
            raise ValueError("bad world size")
        L.lib()
        self.world_size = world_size
        self.config = config or Config.from_env()
        self.device = torch.device(device)
        W = world_size
        self._flag_words = K["TCCL_FLAG_WORDS"]
        self._stage_bytes = int(self.config.stage_mb) << 20
        self.flags = [torch.zeros(self._flag_words, dtype=torch.int32, device=self.device) for _ in range(W)]
        self.tree_bytes = tree_ring_bytes(self.config)
        # one allocation per rank: [staging area (its tail is the small-message region) | double-tree ring]
        self.stages = [torch.empty(self._stage_bytes + self.tree_bytes, dtype=torch.uint8, device=self.device)
                       for _ in range(W)]
        self._zero_tree_ll()
        self.local_states = [torch.zeros(K["TCCL_LOCAL_WORDS"], dtype=torch.int32, device=self.device) for _ in range(W)]
        self.ll_bytes = min(2 << 20, self._stage_bytes // 4)
        self._keep = []
        self.plans = None  # emulated launches are not cached
        self._upload_comms()

    def _zero_tree_ll(self):
        """The small-message tree slots must not start out with bits that look like a flag."""
        for s in self.stages:
            s[self._stage_bytes: self._stage_bytes + K["TCCL_TREE_LL_BYTES"]].zero_()

    def _upload_comms(self):
        W = self.world_size
        arr = (L.Comm * W)()
        for r in range(W):
            c = arr[r]
            c.world, c.rank = W, r
            for p in range(W):
                c.flags[p] = self.flags[p].data_ptr()
                c.stage[p] = self.stages[p].data_ptr()
            c.mc_flags = 0
            c.mc_stage = 0
            c.local = self.local_states[r].data_ptr()
            c.stage_bytes = self._stage_bytes - self.ll_bytes
            c.timeout_ns = self.config.timeout_ns
            c.ll_bytes = self.ll_bytes
            c.tree_bytes = self.tree_bytes
        self._comms_host = arr
        self.comms_dev = self._to_device(arr)

    def _to_device(self, cstruct_array) -> torch.Tensor:
        raw = bytes(cstruct_array)
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)

    # -- tensors
    def empty(self, shape, dtype=torch.bfloat16) -> EmuTensor:
        if isinstance(shape, int):
            shape = (shape,)
        return EmuTensor([torch.empty(*shape, dtype=dtype, device=self.device) for _ in range(self.world_size)])

    def from_parts(self, parts) -> EmuTensor:
        assert len(parts) == self.world_size
        return EmuTensor([p.to(self.device) for p in parts])

    @property
    def local_ranks(self) -> List[int]:
        return list(range(self.world_size))

    @property
    def has_nvls(self) -> bool:
        return False

    def peer_ptrs(self, x: EmuTensor) -> List[int]:
        return [p.data_ptr() for p in x.parts]

    def mc_ptr(self, x) -> int:
        return 0

    def local(self, x: EmuTensor, r: int) -> torch.Tensor:
        return x.parts[r]

    def wrap(self, per_rank):
        return EmuTensor([per_rank[r] for r in range(self.world_size)])

    def stage_ptrs(self) -> List[int]:
        return [s.data_ptr() for s in self.stages]

    def stage_mc(self) -> int:
        return 0

    def ll_ptrs(self) -> List[int]:
        off = self._stage_bytes - self.ll_bytes
        return [s.data_ptr() + off for s in self.stages]

    def ll_mc(self) -> int:
        return 0

    def resident_cta_limit(self, block: int) -> int:
        """CTAs per emulated rank such that all W ranks' CTAs are co-resident
        (assumes one CTA per SM, the worst case of the data kernels)."""
        return max(1, self.num_sms() // self.world_size)

    def max_ctas(self) -> int:
        return min(super().max_ctas(), self.resident_cta_limit(self.config.block))

    def local_copy_ctas(self) -> int:
        return self.max_ctas()  # cooperative launch: stay within what is co-resident

    def prepare(self, name, args_by_rank, grid, block, dtype_code=0):
        W = self.world_size
        first = args_by_rank[0]
        fn = getattr(L.lib(), name)
        l = L.Launch(int(grid), int(block), W, int(dtype_code), None)
        comms = C.c_void_p(self.comms_dev.data_ptr())

        def go():
            # the structs may have been patched since the last call: upload them again
            arr = (type(first) * W)()
            for r in range(W):
                C.memmove(C.byref(arr[r]), C.byref(args_by_rank[r]), C.sizeof(first))
            args_dev = self._to_device(arr)
            self._keep.append(args_dev)
            if len(self._keep) > 64:
                torch.cuda.synchronize(self.device)
                del self._keep[:-1]
            l.stream = torch.cuda.current_stream(self.device).cuda_stream
            rc = fn(comms, C.c_void_p(args_dev.data_ptr()), C.byref(l))
            if rc:
                L.check(rc, name)
            self.launches += 1

        return go

    # -- state
    def last_status(self, rank: int = None):
        def one(r):
            w = self.local_states[r][K["TCCL_LOCAL_STATUS"] : K["TCCL_LOCAL_STATUS"] + K["TCCL_ST_WORDS"]].cpu().tolist()
            return _status_dict([x & 0xFFFFFFFF for x in w])

        if rank is not None:
            return one(rank)
        return [one(r) for r in range(self.world_size)]

    def check(self) -> None:
        for st in self.last_status():
            if st["code"] != 0:
                raise L.TcclTimeout(st)

    def reset(self) -> None:
        torch.cuda.synchronize(self.device)
        for t in self.flags + self.local_states:
            t.zero_()
        self._zero_tree_ll()
        for k in ("_ag_seq", "_stage_user"):  # host-side mirrors of device state
            self.__dict__.pop(k, None)
        torch.cuda.synchronize(self.device)

    def set_timeout_ms(self, ms: float) -> None:
        self.config.timeout_ms = ms
        torch.cuda.synchronize(self.device)
        self._upload_comms()

"""Library configuration: a small dataclass with environment overrides.

The reference hard-codes its constants inside each wrapper (24 CTAs, 16 warps,
world size 8: ``triton_all_gather.py:67-70``,
``triton_double_tree_allreduce.py:254,356``); here they are one object that
every rank must set identically (grid sizes derive from it and the device
barriers pair CTAs by index).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields


def _env(name, default, cast):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    if cast is bool:
        return v not in ("0", "false", "False", "no")
    return cast(v)


@dataclass
class Config:
    timeout_ms: float = 5000.0        # bound of every device-side wait
    max_ctas: int = 0                 # CTAs per collective; 0 = one per SM
    block: int = 512                  # threads per CTA of the data collectives
    nvls_ctas: int = 8                # CTAs of the NVLS two-shot all-reduce (the switch saturates early;
                                      # measured on 8xB200: 4-8 CTAs are best from 8 MiB up, 148 lose a third at 1 GiB)
    pipe_min_bytes: int = 0           # all-reduce: from this size on use the pipelined two-shot (0 = never)
    pipe_ctas: int = 16               # ... its CTAs,
    pipe_reducers: int = 8            # ... warps (of 16 per CTA) that pull; the others push,
    pipe_stages: int = 8              # ... shared-memory stages between the two groups,
    pipe_unroll: int = 4              # ... and 16-byte vectors per reducer thread per stage (2, 4 or 8)
    stage_mb: int = 128               # symmetric staging area per rank
    disable_nvls: bool = False        # never pick a multimem variant
    nvls_barrier: bool = False        # barrier flavour used inside data kernels
    force_variant: str = ""           # e.g. "oneshot_p2p"; empty = size-based choice
    nvls_twoshot_min_bytes: int = 16 * 1024   # all-reduce with a switch and a symmetric destination: two-shot NVLS above this
    push_max_bytes: int = 64 * 1024       # all-reduce: push variant (one barrier, local sum) up to here
    oneshot_max_bytes: int = 512 * 1024   # all-reduce: one-shot up to here, two-shot above
    bulk_min_bytes: int = 64 << 20        # all-reduce at two ranks: from here on the two-shot that moves data with bulk copies (0 = never)
    staged_twoshot: bool = True           # large all-reduce into ordinary memory: two-shot via a cached symmetric buffer
    staged_max_bytes: int = 1 << 30       # ... up to this message size (the buffer is kept per size and dtype)
    tree_chunk_bytes: int = 16 << 20      # double-tree: most bytes per chunk (a chunk = one ring slice per CTA of a tree)
    tree_ctas: int = 36                   # double-tree: CTAs per (tree, direction); 4 x 36 = 144 of 148 SMs
    tree_ll_max_bytes: int = 2 << 20      # double-tree: up to here the flags travel inside the data lines
    tree_pull_min_bytes: int = 1 << 62    # double-tree, chunked kernel: from here on children pull the sum from the parent
                                          # (never by default: measured slower than pushing, 1921 vs 1765 us at 8 ranks, 512 MiB)
    ag_movers: int = 8                    # all-gather -> GEMM: CTAs that move the shard (two alternating groups);
                                          # measured on 8xB200: 8 -> 121 us, 16 -> 123, 24 -> 127, 32 -> 125
    ag_batches: int = 2                   # all-gather -> GEMM on CTA pairs: batches the shard goes out in (one fence each)
    ag_ring: bool = False                 # ... movers send destination by destination (plain stores) instead of in batches to all
    ag_schedule: bool = True              # ... its tiles follow a host-made plan (list scheduling against the rows' arrival)
    ag_pair_tflops: float = 20.0          # ... cost model of that plan: bf16 TFLOP/s of one CTA pair,
    ag_link_gbs: float = 600.0            # ... and GB/s at which the peers' rows arrive
    plan_cache_size: int = 512            # bound launches kept per communicator (least recently used go first)
    debug: bool = False
    debug_shrink_extent: int = 0          # test hook of the TCCL_DEBUG_CHECKS build: claim this many bytes less input

    @classmethod
    def from_env(cls) -> "Config":
        c = cls()
        for f in fields(cls):
            setattr(c, f.name, _env("TCCL_" + f.name.upper(), getattr(c, f.name), type(getattr(c, f.name))))
        return c

    @property
    def timeout_ns(self) -> int:
        return int(self.timeout_ms * 1e6)

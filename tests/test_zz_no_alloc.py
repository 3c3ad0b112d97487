"""The allocation-free entry point (csrc/tccl_noalloc.h), called through its
exported C symbol.

Some users of the library cannot allocate device memory when they need a
reduction — all of it may already belong to a framework's caching allocator, or
they sit on a path where cudaMalloc's device-wide synchronisation is not
acceptable.  ``tccl_allreduce_local_noalloc`` keeps its barrier scratch in a
static device array inside the library instead.  This test runs it twice in a
row on fresh data (the second call meets the scratch exactly as the first left
it) and compares each result with the regular one-shot all-reduce on the same
inputs.  It lives in a file that pytest collects last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, ins, outs, dtype_code, ctas):
    n = len(ins)
    in_arr = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
    out_arr = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    stream = torch.cuda.current_stream().cuda_stream
    fn = lib.tccl_allreduce_local_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_uint64, C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return fn(in_arr, out_arr, n, ins[0].numel(), dtype_code, ctas, C.c_void_p(stream))


@pytest.mark.parametrize("W,dtype,n", [(4, torch.bfloat16, 100003), (8, torch.float32, 1 << 16)])
def test_matches_regular_entry_point_twice(W, dtype, n):
    import tccl_b200 as tccl
    from tccl_b200.config import Config
    from tccl_b200.parallel.emu import EmuWorld
    from tccl_b200.utils import lib as L

    lib = L.lib()
    cfg = Config()
    cfg.stage_mb = 1
    world = EmuWorld(W, config=cfg)
    for call in range(2):
        parts = [torch.randn(n, generator=torch.Generator().manual_seed(100 * call + r)).to(dtype) for r in range(W)]
        x = world.from_parts(parts)
        expect = tccl.all_reduce(x, algo="oneshot_p2p", world=world)
        outs = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(W)]
        rc = _call(lib, list(x.parts), outs, L.DTYPES[dtype], 8)
        assert rc == 0, lib.tccl_error_string(rc)
        torch.cuda.synchronize()
        words = (C.c_uint32 * L.K["TCCL_ST_WORDS"])()
        assert lib.tccl_noalloc_last_status(0, words, None) == 0 and words[0] == 0
        ref = torch.stack([p.float() for p in x.parts]).sum(0)
        tol = {torch.bfloat16: 2 ** -8, torch.float32: 1e-6}[dtype]
        for r in range(W):
            assert bool(((outs[r].float() - ref).abs() <= ref.abs() * tol + 1e-6 * W).all())
            assert torch.equal(outs[r], expect[r])


def test_rejects_sizes_beyond_the_static_scratch():
    from tccl_b200.utils import lib as L

    lib = L.lib()
    xs = [torch.zeros(64, device="cuda") for _ in range(9)]
    ys = [torch.zeros(64, device="cuda") for _ in range(9)]
    assert _call(lib, xs, ys, L.DTYPES[torch.float32], 4) == -L.K["TCCL_ESIZE"]   # 9 ranks > 8
    assert _call(lib, xs[:2], xs[:2], L.DTYPES[torch.float32], 4) == -L.K["TCCL_EINVAL"]  # in place: would race
    assert _call(lib, xs[:2], xs[2:4], L.DTYPES[torch.float32], 17) == -L.K["TCCL_ESIZE"]  # 17 CTAs > 16
    assert b"size" in lib.tccl_error_string(-L.K["TCCL_ESIZE"])

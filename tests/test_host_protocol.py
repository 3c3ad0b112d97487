"""Failure handling of the synchronisation protocols, tested on the host: CPU
processes run the C++ twin of the device protocol over shared memory, and the
faults (a lost signal, a stalled rank, a rank that stops or never joins) are
injected there.  Every wait is bounded, so a failed peer turns into a TIMEOUT
status that names the peer — never into a hang."""
import time

import numpy as np
import pytest

from tccl_b200.utils.hostproto import run_ranks


def test_barrier_many_rounds():
    res, _ = run_ranks(4, "barrier", faults={r: {"rounds": 200} for r in range(4)})
    assert all(v["ok"] == 1 and v["status"]["code"] == 0 for v in res.values())


@pytest.mark.parametrize("pull_down", [0, 1])
@pytest.mark.parametrize("W", [2, 4, 8])
def test_tree_allreduce_on_cpu_ranks(W, pull_down):
    n = 1 << 14
    xs = [np.random.default_rng(r).standard_normal(n).astype(np.float32) for r in range(W)]
    res, outs = run_ranks(W, "tree", numel=n, inputs=xs,
                          faults={r: {"chunk": 1 << 9, "pull_down": pull_down} for r in range(W)})
    assert all(v["ok"] == 1 for v in res.values()), res
    ref = np.sum(np.stack(xs).astype(np.float64), 0)
    for o in outs:
        np.testing.assert_allclose(o, ref, rtol=1e-5, atol=1e-5)
        assert np.array_equal(o, outs[0])


def test_lost_signal_becomes_a_timeout_that_names_the_peer():
    t0 = time.time()
    res, _ = run_ranks(4, "barrier", timeout_ms=300, faults={1: {"drop_signal_to": 2}})
    assert time.time() - t0 < 20
    st = res[2]["status"]
    assert res[2]["ok"] == 0 and st["code"] == 1 and st["where"] == "TCCL_W_BARRIER" and st["peer"] == 1 and st["aborted"]
    for r in (0, 1, 3):  # a single round: the others did get every signal
        assert res[r]["ok"] == 1


def test_stalled_rank_within_the_limit_is_not_a_failure():
    res, _ = run_ranks(4, "barrier", timeout_ms=3000, faults={3: {"stall_ms": 300}})
    assert all(v["ok"] == 1 for v in res.values())


def test_rank_that_never_joins():
    res, _ = run_ranks(4, "barrier", timeout_ms=300, faults={2: {"never_join": True}})
    for r in (0, 1, 3):
        st = res[r]["status"]
        assert res[r]["ok"] == 0 and st["code"] == 1 and st["peer"] == 2


@pytest.mark.parametrize("pull_down", [0, 1])
def test_rank_that_stops_mid_all_reduce(pull_down):
    """Rank 2 stops after three chunks: its tree neighbours time out in the up or
    down phase, everybody returns, nobody hangs."""
    W, n = 4, 1 << 14
    xs = [np.ones(n, np.float32) * r for r in range(W)]
    t0 = time.time()
    res, _ = run_ranks(W, "tree", numel=n, inputs=xs, timeout_ms=400,
                       faults={r: ({"chunk": 1 << 9, "pull_down": pull_down, "stop_after_chunk": 3} if r == 2
                                   else {"chunk": 1 << 9, "pull_down": pull_down}) for r in range(W)})
    assert time.time() - t0 < 30
    failed = [r for r in range(W) if res[r]["ok"] == 0]
    assert failed, res
    wheres = {res[r]["status"]["where"] for r in failed if res[r]["status"]["code"]}
    assert wheres & {"TCCL_W_TREE_UP", "TCCL_W_TREE_DOWN", "TCCL_W_BARRIER"}


@pytest.mark.parametrize("W", [2, 3, 4, 8])
def test_protocol_is_race_free_under_thread_sanitizer(W):
    """Ranks (and CTAs) as threads of one process, instrumented with ThreadSanitizer: every plain
    access of the data buffers must be ordered by the release/acquire flags.  Covers the barrier,
    the double-tree pipeline (pushed and pulled way down), the flag-in-line tree (slot depth 4 and 1),
    the GEMM -> reduce-scatter tile flags
    (deferred release, final phase, epoch hand-over across calls), the all-gather -> GEMM arrival
    flags, the push all-reduce with changing sizes and grids, the barrier-free CTA-pair forms of both
    fused GEMM ops (two alternating halves, 40 calls with the ranks drifting apart; batched and
    ring-ordered movers) and the stage pipeline of the bulk-copy all-reduce."""
    import subprocess

    from tccl_b200.utils import build as B

    try:
        exe = B.build_host_tsan()
    except RuntimeError as e:  # no libtsan on this machine
        pytest.skip(str(e)[:200])
    r = subprocess.run([str(exe), str(W), str(1 << 13), str(1 << 8)], capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert "ThreadSanitizer" not in out, out[-3000:]
    assert r.returncode == 0, out[-2000:]


def test_thread_sanitizer_flags_the_size_dependent_push_layout():
    """The push all-reduce's slot layout must not depend on the message: with a slot size equal to
    the message and the half taken from a CTA's own barrier epoch, calls of alternating size and
    grid let a fast rank overwrite bytes a slow peer is still summing.  The model keeps that variant
    so that this test can show ThreadSanitizer (or the sum check) catching it; the layout the kernel
    uses runs clean in test_protocol_is_race_free_under_thread_sanitizer."""
    import subprocess

    from tccl_b200.utils import build as B

    try:
        exe = B.build_host_tsan()
    except RuntimeError as e:
        pytest.skip(str(e)[:200])
    r = subprocess.run([str(exe), "push-broken-variant", "4"], capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert "ThreadSanitizer: data race" in out or r.returncode != 0, out[-2000:]


def test_thread_sanitizer_flags_an_output_stage_freed_before_its_copies_have_read_it():
    """The bulk-copy all-reduce hands its sums to the copy engine from shared-memory stages; a stage
    may be refilled only when the copies issued from it have READ it (cp.async.bulk.wait_group.read),
    not when they were issued.  The model keeps the early release as a variant, with a copy-engine
    thread that runs behind the issuer, so that ThreadSanitizer (or the sum check) is seen to catch
    it; the order the kernel uses runs clean in test_protocol_is_race_free_under_thread_sanitizer."""
    import subprocess

    from tccl_b200.utils import build as B

    try:
        exe = B.build_host_tsan()
    except RuntimeError as e:
        pytest.skip(str(e)[:200])
    r = subprocess.run([str(exe), "bulk-broken-variant", "4"], capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert "ThreadSanitizer: data race" in out or r.returncode != 0, out[-2000:]


def test_thread_sanitizer_flags_a_single_gather_buffer_without_a_barrier():
    """The all-gather -> GEMM pair kernel has no entry barrier because its gathered buffer has two
    halves that alternate from call to call; with ONE buffer a rank that is a call ahead overwrites
    rows a slower peer is still reading.  The model keeps that variant so that ThreadSanitizer (or the
    value check) is seen to catch it; the two-halves scheme runs clean, with batched and with
    ring-ordered movers, in test_protocol_is_race_free_under_thread_sanitizer."""
    import subprocess

    from tccl_b200.utils import build as B

    try:
        exe = B.build_host_tsan()
    except RuntimeError as e:
        pytest.skip(str(e)[:200])
    r = subprocess.run([str(exe), "ag-pair-broken-variant", "4"], capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert "ThreadSanitizer: data race" in out or r.returncode != 0, out[-2000:]


def test_thread_sanitizer_flags_a_single_staging_half_without_a_barrier():
    """Same obligation for the GEMM -> reduce-scatter pair kernel: its staging area alternates between
    two halves instead of opening with a barrier; with ONE half a rank that is a call ahead overwrites
    partials a slower peer is still summing.  The kept variant must be caught; the two-halves scheme
    runs clean in test_protocol_is_race_free_under_thread_sanitizer (40 calls, ranks drifting apart)."""
    import subprocess

    from tccl_b200.utils import build as B

    try:
        exe = B.build_host_tsan()
    except RuntimeError as e:
        pytest.skip(str(e)[:200])
    r = subprocess.run([str(exe), "rs-pair-broken-variant", "4"], capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert "ThreadSanitizer: data race" in out or r.returncode != 0, out[-2000:]

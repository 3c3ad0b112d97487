"""Host-side failure detection with gloo ranks on the CPU: a rank that leaves
between steps is seen through the store before the next launch; a rank that
goes silent is seen after the staleness limit; and a short process-group
timeout turns a collective with a missing rank into an error, not a hang."""
import datetime
import os
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tccl_b200.utils.health import PeerLost, PeerMonitor


def _worker(rank, world, port, scenario, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    store = dist.distributed_c10d._get_default_store()
    mon = PeerMonitor(store, rank, world, stale_s=1.0)
    out = {"rank": rank, "steps": 0, "lost": None, "collective_error": None}
    try:
        for step in range(6):
            if scenario == "leave" and rank == 1 and step == 3:
                mon.leave()  # between steps: nothing of this rank is in flight
                break
            if scenario == "silent" and rank == 1 and step == 3:
                time.sleep(4.0)  # stops beating without saying so
                break
            mon.beat()
            time.sleep(0.05)
            if scenario in ("leave", "silent"):
                if step >= 3:
                    deadline = time.time() + 3.0
                    while time.time() < deadline:  # learn of it on the host, before the next launch
                        mon.beat()  # this rank is alive and says so while it waits
                        try:
                            mon.check()
                        except PeerLost as e:
                            out["lost"] = e.ranks
                            break
                        time.sleep(0.1)
                    break
            if scenario == "pg_timeout" and step == 2:
                if rank == 1:
                    time.sleep(6.0)  # never joins the collective in time
                    break
                try:
                    t = torch.ones(4)
                    dist.all_reduce(t)
                except Exception as e:  # noqa: BLE001
                    out["collective_error"] = type(e).__name__
                break
            t = torch.ones(4) * rank
            dist.all_reduce(t)
            out["steps"] += 1
    finally:
        q.put(out)
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(scenario, world=3):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300)
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        o = q.get(timeout=60)
        res[o["rank"]] = o
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()  # the exact child started above
    return res


def test_rank_that_leaves_between_steps_is_seen_on_the_host():
    res = _run("leave")
    assert res[0]["lost"] == [1] and res[2]["lost"] == [1]
    assert res[0]["steps"] == 3


def test_silent_rank_is_reported_after_the_staleness_limit():
    res = _run("silent")
    assert res[0]["lost"] == [1] and res[2]["lost"] == [1]


def test_short_process_group_timeout_ends_the_collective_with_an_error():
    res = _run("pg_timeout")
    assert res[0]["collective_error"] is not None and res[2]["collective_error"] is not None

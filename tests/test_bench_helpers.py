"""Timing / roofline helpers and the clock sampler's summary, without a GPU."""
import importlib.util
import os

from tccl_b200.utils.clocks import ClockSampler
from tccl_b200.utils.timing import summarize

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    return spec, mod


def test_summarize_percentiles():
    st = summarize([0.010 + 0.001 * i for i in range(100)])  # milliseconds
    assert abs(st["p50_us"] - 59.5) < 1.0 and st["min_us"] == 10.0 and st["iters"] == 100
    assert st["p10_us"] < st["p50_us"] < st["p90_us"]


def test_clock_summary_uses_only_samples_inside_the_marks():
    s = ClockSampler()
    s.samples = [(0.5, 1200.0, 1965.0, 0x4, 500.0), (1.5, 1900.0, 1965.0, 0x0, 900.0), (1.6, 1950.0, 1965.0, 0x4, 950.0),
                 (3.0, 300.0, 1965.0, 0x40, 100.0)]
    s._t0, s._t1 = 1.0, 2.0
    out = s.summary()
    assert out["samples"] == 2 and out["sm_mhz"] == 1925.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 950.0
    s._t0, s._t1 = 10.0, 11.0  # nothing inside: fall back to everything recorded
    assert s.summary()["samples"] == 4 and "hw_thermal_slowdown" in s.summary()["reasons"]


def test_nvlink_traffic_model_of_the_sweep():
    src = open(os.path.join(ROOT, "bench", "sweep.py")).read()
    ns = {}
    start = src.index("def nvlink_bytes_in")
    end = src.index("def main()")
    exec(src[start:end], ns)  # the two pure functions only (the module itself needs torch.distributed + CUDA)
    f, best = ns["nvlink_bytes_in"], ns["best_possible_bytes_in"]
    S, W = 1 << 20, 8
    assert f("allreduce", "oneshot_p2p", W, S) == 7 * S
    assert f("allreduce", "twoshot_p2p", W, S) == 2 * 7 * S // 8
    assert f("allreduce", "twoshot_nvls", W, S) == S + S // 8
    assert f("allgather", "pull", W, S) == 7 * S and f("reducescatter", "p2p", W, S) == 7 * S // 8
    assert f("allreduce", "tree", 1, S) == 0
    assert best("allreduce", W, S, True) == S and best("allreduce", W, S, False) == 2 * 7 * S // 8

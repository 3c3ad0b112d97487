"""Sample SM clocks and throttle reasons while a timed region runs.

Read-only: nothing here changes a GPU setting.  NVML (through ``pynvml``) is
polled from a thread every few milliseconds, so that even a timed region of a
few milliseconds gets samples; ``nvidia-smi`` is the fallback when the NVML
binding is missing.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import List, Optional

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

# NVML clocks-event-reason bits
_REASONS = {
    0x0000000000000004: "sw_power_cap",
    0x0000000000000008: "hw_slowdown",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
}


class ClockSampler:
    """``with ClockSampler(uuids) as s: ...; s.mark_start(); ...; s.mark_end()``.
    ``summary()`` covers the samples between the marks (all samples if unmarked)."""

    def __init__(self, gpu_uuids: Optional[List[str]] = None, period_ms: float = 2.0):
        self.gpu_uuids, self.period = gpu_uuids, period_ms / 1e3
        self.samples = []  # (t, sm_mhz, max_mhz, reasons_mask, power_w)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._t0: Optional[float] = None
        self._t1: Optional[float] = None
        self._smi: Optional[subprocess.Popen] = None
        self.backend = "none"

    # -- NVML path
    def _nvml_handles(self):
        import pynvml as N

        N.nvmlInit()
        hs = []
        if self.gpu_uuids:
            for u in self.gpu_uuids:
                u = u if u.startswith("GPU-") else "GPU-" + u
                hs.append(N.nvmlDeviceGetHandleByUUID(u))
        else:
            for i in range(N.nvmlDeviceGetCount()):
                hs.append(N.nvmlDeviceGetHandleByIndex(i))
        return N, hs

    def _poll_nvml(self, N, hs):
        maxes = [N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM) for h in hs]
        get_reasons = getattr(N, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            N, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            now = time.perf_counter()
            for h, mx in zip(hs, maxes):
                try:
                    sm = N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM)
                    rs = int(get_reasons(h))
                    pw = N.nvmlDeviceGetPowerUsage(h) / 1e3
                except Exception:  # noqa: BLE001 - a failed read is just a missing sample
                    continue
                self.samples.append((now, float(sm), float(mx), rs, pw))
            self._stop.wait(self.period)

    # -- nvidia-smi fallback
    def _poll_smi(self):
        for line in self._smi.stdout:
            r = [c.strip() for c in line.split(",")]
            if len(r) < 9:
                continue
            try:
                sm, mx = float(r[1]), float(r[2])
            except ValueError:
                continue
            mask = 0
            for bit, col in ((0x8, 5), (0x40, 6), (0x20, 7), (0x4, 8)):
                if r[col].lower().startswith("active"):
                    mask |= bit
            try:
                pw = float(r[3])
            except ValueError:
                pw = 0.0
            self.samples.append((time.perf_counter(), sm, mx, mask, pw))

    def __enter__(self):
        try:
            N, hs = self._nvml_handles()
            self._thread = threading.Thread(target=self._poll_nvml, args=(N, hs), daemon=True)
            self.backend = "nvml"
        except Exception:  # noqa: BLE001 - no NVML binding: fall back to the CLI
            try:
                self._smi = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self._thread = threading.Thread(target=self._poll_smi, daemon=True)
                self.backend = "nvidia-smi"
            except OSError:
                self._thread = None
        if self._thread:
            self._thread.start()
        return self

    def mark_start(self):
        self._t0 = time.perf_counter()

    def mark_end(self):
        self._t1 = time.perf_counter()

    def __exit__(self, *exc):
        self._stop.set()
        if self._smi is not None:
            self._smi.terminate()  # the exact child we started
            try:
                self._smi.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._smi.kill()
        if self._thread:
            self._thread.join(timeout=2)
        return False

    def summary(self) -> dict:
        rows = self.samples
        if self._t0 is not None:
            t1 = self._t1 if self._t1 is not None else float("inf")
            inside = [s for s in rows if self._t0 <= s[0] <= t1]
            rows = inside or rows  # a region shorter than the poll period: use what there is
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "backend": self.backend}
        mask = 0
        for s in rows:
            mask |= s[3]
        return {"sm_mhz": statistics.median(s[1] for s in rows), "sm_max_mhz": max(s[2] for s in rows),
                "reasons": sorted(name for bit, name in _REASONS.items() if mask & bit),
                "power_w_max": round(max(s[4] for s in rows), 1), "samples": len(rows), "backend": self.backend}

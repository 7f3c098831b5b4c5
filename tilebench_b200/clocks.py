"""SM clock and throttle-reason sampling through NVML while a timed region runs (read-only: nothing here
changes a clock, a power limit or any other device setting)."""
from __future__ import annotations

import statistics
import threading
import time

#: NVML clock-event reason bits that matter for a benchmark number.
REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
           0x80: "hw_power_brake_slowdown"}


class ClockSampler:
    """Polls one GPU every `period_s` while `busy(True)` is in force; `stop()` / `snapshot()` give the median SM
    clock, the maximum SM clock and every reason seen.  Without NVML it stays empty."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples, self.reasons, self.power_w, self.max_mhz = [], set(), [], None
        self._period = period_s
        self._stop = threading.Event()
        self._busy = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            if self._busy.is_set():
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                    mask = reasons_fn(self._h)
                    for bit, name in REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                    self.power_w.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                except Exception:
                    pass
            time.sleep(self._period)

    def start(self):
        if self._nv is not None and self._thread is None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def busy(self, on: bool):
        (self._busy.set if on else self._busy.clear)()

    def mark(self) -> int:
        """Index of the next sample; pass it to snapshot() to summarise only what came after."""
        return len(self.samples)

    def snapshot(self, since: int = 0) -> dict:
        s = self.samples[since:]
        p = self.power_w[since:]
        return {"sm_mhz": statistics.median(s) if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s), "power_w_max": max(p) if p else None}

    def stop(self) -> dict:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)
        return self.snapshot()

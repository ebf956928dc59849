"""Read-only sampling of GPU clocks and throttle reasons during a timed region (NVML; nothing is set)."""
from __future__ import annotations

import statistics
import threading
import time
from typing import Dict, List, Optional

# NVML clocks-event-reason bits
_REASONS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
    0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
}


class ClockSampler:
    def __init__(self, index: int = 0, period_s: float = 0.2):
        self.index, self.period = index, period_s
        self.sm: List[int] = []
        self.power: List[float] = []
        self.reason_bits = 0
        self.sm_max: Optional[int] = None
        self._stop = threading.Event()
        self._thr: Optional[threading.Thread] = None
        self.error: Optional[str] = None

    def _run(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self._stop.is_set():
                self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                try:
                    self.power.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)) & ~0x1
                except Exception:
                    pass
                self._stop.wait(self.period)
            pynvml.nvmlShutdown()
        except Exception as exc:  # no NVML: report, do not fail the benchmark
            self.error = repr(exc)

    def __enter__(self):
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=2)

    def summary(self) -> Dict:
        reasons = [name for bit, name in _REASONS.items() if self.reason_bits & bit]
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.sm_max, "reasons": reasons,
               "samples": len(self.sm), "power_w_max": max(self.power) if self.power else None}
        if self.error:
            out["error"] = self.error
        return out

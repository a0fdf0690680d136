"""SM clock and throttle reasons while a measurement runs (NVML, reading only)."""
from __future__ import annotations

import threading
import time


class ClockSampler:
    """Reads SM clock and throttle reasons through NVML every 5 ms while ``on`` is set.
    Reading only: nothing about the GPU is changed."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, index: int = 0):
        self.samples, self.reasons, self.on, self._stop = [], set(), False, False
        self.times = []                    # time.perf_counter() of each sample
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception as e:          # noqa: BLE001
            self.nv = None
            self.error = str(e)

    def _run(self):
        nv = self.nv
        while not self._stop:
            if self.on:
                try:
                    self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                    self.times.append(time.perf_counter())
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:       # noqa: BLE001
                    pass
            time.sleep(0.005)

    def median_between(self, t0: float, t1: float):
        """Median SM clock over the samples taken between two ``time.perf_counter()`` readings."""
        s = sorted(m for m, t in zip(self.samples, self.times) if t0 <= t <= t1)
        return s[len(s) // 2] if s else None

    def summary(self):
        self._stop = True
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": getattr(self, "error", "")}
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}

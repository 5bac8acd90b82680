"""Read-only sampling of GPU clocks and throttle reasons during a timed region.

Uses NVML queries only (nothing here changes a clock, a power limit or any other device
setting).
"""
from __future__ import annotations

import statistics
import threading
from typing import List, Optional

_REASONS = {
    0x0000000000000002: "applications_clocks_setting",
    0x0000000000000004: "sw_power_cap",
    0x0000000000000008: "hw_slowdown",
    0x0000000000000010: "sync_boost",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000080: "hw_power_brake_slowdown",
    0x0000000000000100: "display_clock_setting",
}


class ClockSampler:
    def __init__(self, device_index: int = 0, period_s: float = 0.2):
        self.idx = device_index
        self.period = period_s
        self.samples: List[int] = []
        self.power: List[float] = []
        self.reason_bits = 0
        self.sm_max = None
        self._stop = threading.Event()
        self._th: Optional[threading.Thread] = None
        self._ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self._ok = True
        except Exception:
            self._ok = False

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                                        if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                                        else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._ok:
            self._th = threading.Thread(target=self._run, daemon=True)
            self._th.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=2.0)
        reasons = [name for bit, name in _REASONS.items() if self.reason_bits & bit]
        return {
            "sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.sm_max,
            "reasons": reasons,
            "power_w_max": round(max(self.power), 1) if self.power else None,
            "samples": len(self.samples),
        }

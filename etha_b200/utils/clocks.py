"""Read-only sampling of GPU clocks and throttle reasons while a benchmark runs (NVML queries only)."""

from __future__ import annotations

import statistics
import threading
import time

_REASONS = {
    0x1: "gpu_idle",
    0x2: "applications_clocks_setting",
    0x4: "sw_power_cap",
    0x8: "hw_slowdown",
    0x10: "sync_boost",
    0x20: "sw_thermal_slowdown",
    0x40: "hw_thermal_slowdown",
    0x80: "hw_power_brake_slowdown",
    0x100: "display_clock_setting",
}


class ClockSampler:
    """Background thread polling SM clock, power and clock-event reasons of one GPU."""

    def __init__(self, device_index: int = 0, period_s: float = 0.01):
        self.device_index = device_index
        self.period_s = period_s
        self.samples: list[tuple[int, int, float]] = []  # (sm_mhz, reasons bitmask, watts)
        self.sm_max_mhz = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.sm_max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._ok = True
        except Exception:
            self._ok = False

    def _loop(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                try:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                except Exception:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                except Exception:
                    watts = 0.0
                self.samples.append((mhz, reasons, watts))
            except Exception:
                pass
            time.sleep(self.period_s)

    def start(self) -> "ClockSampler":
        if self._ok:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max_mhz or None, "reasons": [], "samples": 0}
        mask = 0
        for _, r, _ in self.samples:
            mask |= r
        reasons = [name for bit, name in _REASONS.items() if mask & bit and name != "gpu_idle"]
        return {
            "sm_mhz": int(statistics.median(s[0] for s in self.samples)),
            "sm_max_mhz": self.sm_max_mhz,
            "reasons": reasons,
            "samples": len(self.samples),
            "power_w_max": round(max(s[2] for s in self.samples), 1),
        }

"""Read-only sampling of SM clocks and throttle reasons while a benchmark runs."""

from __future__ import annotations

import statistics
import threading

_REASONS = {
    "sw_power_cap": 0x4,
    "hw_slowdown": 0x8,
    "sync_boost": 0x10,
    "sw_thermal_slowdown": 0x20,
    "hw_thermal_slowdown": 0x40,
    "hw_power_brake_slowdown": 0x80,
    "display_clock_setting": 0x100,
}


class ClockSampler:
    """Background NVML reader (never writes any GPU setting)."""

    def __init__(self, device_index=0, interval_s=0.05):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._interval = interval_s
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread = None
        self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception as error:  # NVML missing: report that instead of failing the benchmark
            self.error = repr(error)

    def _loop(self):
        nvml = self._nvml
        while not self._stop.is_set():
            if self._paused.is_set():
                self._stop.wait(self._interval)
                continue
            try:
                self.samples.append(nvml.nvmlDeviceGetClockInfo(self._handle, nvml.NVML_CLOCK_SM))
                getter = getattr(nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nvml.nvmlDeviceGetCurrentClocksThrottleReasons
                bits = getter(self._handle)
                for name, bit in _REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self._interval)

    def __enter__(self):
        if self._handle is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def pause(self):
        self._paused.set()

    def resume(self):
        self._paused.clear()

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return False

    def summary(self):
        if self._handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": getattr(self, "error", "nvml unavailable")}
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}

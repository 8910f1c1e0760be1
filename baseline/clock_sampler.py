"""Read-only sampler of one GPU's SM clock, power draw and clock-event reasons for the reference arm.

Self-contained on purpose: the reference arm imports nothing of the ``universal_gemm_b200`` package.  A thread
polls NVML every few milliseconds between ``start()`` and ``stop()``; no clock, power or mode setting is touched.
"""
from __future__ import annotations

import statistics
import threading
import time

_REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: float = 5.0):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._samples: list[tuple[float, float, int]] = []
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._max: float | None = None

    def start(self) -> bool:
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            return False

        def poll() -> None:
            while not self._stop.is_set():
                try:
                    sm = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                    power = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                    try:
                        reasons = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                    except Exception:  # noqa: BLE001
                        reasons = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                    self._samples.append((sm, power, reasons))
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(self.period_ms / 1000.0)

        self._thread = threading.Thread(target=poll, daemon=True)
        self._thread.start()
        return True

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self._samples:
            return {"sm_mhz": None, "sm_max_mhz": self._max, "reasons": ["no samples"], "samples": 0}
        pmax = max(p for _, p, _ in self._samples)
        busy = [s for s in self._samples if s[1] >= 0.6 * pmax] or self._samples
        mask = 0
        for _, _, r in busy:
            mask |= r
        return {"sm_mhz": statistics.median(s for s, _, _ in busy), "sm_max_mhz": self._max, "power_w_max": pmax,
                "reasons": sorted(name for bit, name in _REASONS.items() if mask & bit),
                "samples": len(self._samples), "samples_under_load": len(busy), "source": "nvml"}

"""Measurement helpers shared by ``bench.py`` and the benchmark suite: device timing with
CUDA events (max over ranks) and a background sampler of SM clocks / throttle reasons."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time

import torch

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU between ``start()`` and ``stop()``.

    Uses NVML queries from a thread every few milliseconds (timed regions of a multi-GPU GEMM are only tens of
    milliseconds long); falls back to ``nvidia-smi -lms 200`` when NVML cannot be loaded.  Read-only: no clock,
    power or mode setting is touched."""

    _REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int = 0, period_ms: float = 3.0):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._samples: list[tuple[float, float, int]] = []
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._nvml = None
        self._max = None
        self._smi: _SmiSampler | None = None

    def start(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._nvml = (pynvml, handle)
        except Exception:  # noqa: BLE001
            self._smi = _SmiSampler(self.gpu_index)
            self._smi.start()
            return

        def poll():
            nv, h = self._nvml
            while not self._stop.is_set():
                try:
                    sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    power = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                    try:
                        reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                    except Exception:  # noqa: BLE001
                        reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    self._samples.append((sm, power, reasons))
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(self.period_ms / 1000.0)

        self._thread = threading.Thread(target=poll, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._smi is not None:
            return self._smi.stop()
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
                "reasons": sorted(name for bit, name in self._REASONS.items() if mask & bit),
                "samples": len(self._samples), "samples_under_load": len(busy), "source": "nvml"}


class _SmiSampler:
    """``nvidia-smi`` fallback of :class:`ClockSampler` (one sample every 200 ms)."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc: subprocess.Popen | None = None
        self._lines: list[str] = []
        self._thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump():
            assert self._proc is not None and self._proc.stdout is not None
            for line in self._proc.stdout:
                self._lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(self.period_ms / 1000.0 * 1.5)
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=2)
        sm, sm_max, power = [], [], []
        reasons: set[str] = set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self._lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "samples": 0}
        busy = [s for s, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(sm_max), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def max_over_ranks(value: float, device: torch.device) -> float:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_all(world) -> None:
    """Barrier + device synchronise on both sides of a timed region."""
    if world.is_cuda:
        torch.cuda.synchronize(world.device)
    world.barrier()
    if world.is_cuda:
        torch.cuda.synchronize(world.device)

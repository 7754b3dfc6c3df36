"""Sample GPU clocks, power and throttle reasons while a benchmark's timed region runs: through
NVML (`pynvml`, every 20 ms from a thread) when it is importable and initialises, else with an
`nvidia-smi -lms` subprocess. Read-only: nothing here changes a GPU setting."""
from __future__ import annotations

import os
import statistics
import subprocess
import threading
from typing import Dict, List, Optional

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
           "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
           "clocks_event_reasons.sw_power_cap")
_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")


# NVML clocks-event (throttle) reason bits, nvml.h
_NVML_REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))


class ClockSampler:
    """`with ClockSampler(gpu_index) as c: ...; c.summary()`"""

    def __init__(self, index: int = 0, period_ms: int = 200, nvml_period_ms: int = 20):
        self.index = index
        self.period_ms = period_ms
        self.nvml_period_ms = nvml_period_ms
        self.samples: List[List[str]] = []
        self._proc: Optional[subprocess.Popen] = None
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.source = "none"

    def _start_nvml(self) -> bool:
        """Sampling thread on NVML; False if NVML is not usable here."""
        try:
            import pynvml

            pynvml.nvmlInit()
            # NVML numbers devices like nvidia-smi; CUDA_VISIBLE_DEVICES remaps CUDA ordinals only.
            index = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    index = int(ids[self.index])
            h = pynvml.nvmlDeviceGetHandleByIndex(index)
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            reasons_fn(h)
        except Exception:
            return False

        def loop():
            while not self._stop.is_set():
                try:
                    sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                    pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                    bits = int(reasons_fn(h))
                    flags = ["Active" if bits & bit else "Not Active" for bit, _ in _NVML_REASONS]
                    self.samples.append([str(index), str(sm), str(mx), f"{pw:.2f}"] + flags)
                except Exception:
                    pass
                self._stop.wait(self.nvml_period_ms / 1000.0)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        self.source = "nvml"
        return True

    def __enter__(self):
        if self._start_nvml():
            return self
        self.source = "nvidia-smi"
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            assert self._proc is not None and self._proc.stdout is not None
            for line in self._proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 8:
                    self.samples.append(parts)

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def summary(self) -> Dict:
        sm, mx, pw = [], [], []
        reasons = set()
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
                pw.append(float(s[3]))
            except ValueError:
                continue
            for name, v in zip(_REASONS, s[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(pw), "reasons": sorted(reasons),
                "samples": len(sm), "source": self.source}

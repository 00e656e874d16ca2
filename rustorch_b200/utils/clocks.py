"""Read-only sampling of GPU clocks and throttle reasons while a benchmark runs (NVML).

Nothing here changes a GPU setting; it only reads ``clocks.sm``, ``clocks.max.sm`` and the
active clock-event reasons, the same fields as
``nvidia-smi --query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active``.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import List, Optional

_REASONS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
    0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
    0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
}


class ClockSampler:
    def __init__(self, device_index: int = 0, period_s: float = 0.2):
        self.device_index = device_index
        self.period_s = period_s
        self.samples: List[int] = []
        self.reason_bits = 0
        self.sm_max: Optional[int] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._nvml = None
        self._handle = None

    def _init_nvml(self) -> bool:
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            return True
        except Exception:  # noqa: BLE001
            self._nvml = None
            return False

    def _sample_nvml(self) -> None:
        n = self._nvml
        self.samples.append(int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
        try:
            self.reason_bits |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
        except Exception:  # noqa: BLE001
            try:
                self.reason_bits |= int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
            except Exception:  # noqa: BLE001
                pass

    def _sample_smi(self) -> None:
        try:
            out = subprocess.run(
                ["nvidia-smi", f"--id={self.device_index}",
                 "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active",
                 "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
            parts = [p.strip() for p in out.strip().split(",")]
            self.samples.append(int(parts[0]))
            self.sm_max = int(parts[1])
            self.reason_bits |= int(parts[2], 16)
        except Exception:  # noqa: BLE001
            pass

    def _run(self) -> None:
        use_nvml = self._init_nvml()
        while not self._stop.is_set():
            try:
                self._sample_nvml() if use_nvml else self._sample_smi()
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period_s)

    def start(self) -> "ClockSampler":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        reasons = [name for bit, name in _REASONS.items()
                   if self.reason_bits & bit and name != "gpu_idle"]
        return {
            "sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.sm_max,
            "reasons": reasons,
            "samples": len(self.samples),
        }

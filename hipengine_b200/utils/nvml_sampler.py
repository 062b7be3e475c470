"""Background sampler of device memory, clocks, power and throttle reasons over NVML (read-only).

The role of the reference's VRAM sampler (``hipengine/util/amdgpu_vram.py``: a thread that samples VRAM / GTT from
sysfs while a benchmark runs and reports peaks) on NVIDIA hardware.  Only getters are called: nothing here sets a
clock, a power limit or any other device setting.  The NVML module is injectable, so the sampler is tested on a CPU
box against a fake.

    with NvmlSampler(device_index=0, interval_s=0.2) as s:
        run_benchmark()
    print(s.summary())     # peak memory, median / min SM clock, median power, throttle reasons seen
"""
from __future__ import annotations

import statistics
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

# bit -> name of nvmlClocksEventReasons* (the ones a benchmark must report; NVML's values)
REASON_BITS = {
    0x0000000000000001: "gpu_idle",
    0x0000000000000002: "applications_clocks_setting",
    0x0000000000000004: "sw_power_cap",
    0x0000000000000008: "hw_slowdown",
    0x0000000000000010: "sync_boost",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000080: "hw_power_brake_slowdown",
    0x0000000000000100: "display_clock_setting",
}
REJECTING = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")
NVML_CLOCK_SM = 1


@dataclass
class Sample:
    t: float
    mem_used: int
    mem_total: int
    sm_mhz: Optional[int]
    power_w: Optional[float]
    reasons: int


def decode_reasons(mask: int) -> List[str]:
    return [name for bit, name in sorted(REASON_BITS.items()) if mask & bit and name != "gpu_idle"]


@dataclass
class NvmlSampler:
    device_index: int = 0
    interval_s: float = 0.2
    nvml: Any = None                       # module with the pynvml functions; imported on start when None
    samples: List[Sample] = field(default_factory=list)

    def __post_init__(self) -> None:
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._handle = None
        self._max_sm: Optional[int] = None
        self.error: Optional[str] = None

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "NvmlSampler":
        try:
            if self.nvml is None:
                import pynvml
                self.nvml = pynvml
            self.nvml.nvmlInit()
            self._handle = self.nvml.nvmlDeviceGetHandleByIndex(self.device_index)
            try:
                self._max_sm = int(self.nvml.nvmlDeviceGetMaxClockInfo(self._handle, NVML_CLOCK_SM))
            except Exception:
                self._max_sm = None
        except Exception as exc:           # no driver, no device: the sampler reports that instead of raising
            self.error = f"{type(exc).__name__}: {exc}"
            return self
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, name="nvml-sampler", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)
            self._thread = None
        if self._handle is not None:
            try:
                self.nvml.nvmlShutdown()
            except Exception:
                pass
            self._handle = None

    def __enter__(self) -> "NvmlSampler":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()

    # ------------------------------------------------------------------ sampling
    def sample_once(self) -> Optional[Sample]:
        n, h = self.nvml, self._handle
        if h is None:
            return None
        mem = n.nvmlDeviceGetMemoryInfo(h)
        get = lambda fn, *a: self._try(fn, h, *a)
        sm = get(n.nvmlDeviceGetClockInfo, NVML_CLOCK_SM)
        mw = get(n.nvmlDeviceGetPowerUsage)
        fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        rs = self._try(fn, h) if fn is not None else None
        s = Sample(time.time(), int(mem.used), int(mem.total), None if sm is None else int(sm),
                   None if mw is None else float(mw) / 1000.0, int(rs or 0))
        self.samples.append(s)
        return s

    @staticmethod
    def _try(fn, *a):
        try:
            return fn(*a)
        except Exception:
            return None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self.sample_once()
            except Exception as exc:
                self.error = f"{type(exc).__name__}: {exc}"
                return
            self._stop.wait(self.interval_s)

    # ------------------------------------------------------------------ report
    def summary(self) -> Dict[str, Any]:
        if not self.samples:
            return {"samples": 0, "error": self.error or "no samples"}
        sm = [s.sm_mhz for s in self.samples if s.sm_mhz is not None]
        pw = [s.power_w for s in self.samples if s.power_w is not None]
        mask = 0
        for s in self.samples:
            mask |= s.reasons
        reasons = decode_reasons(mask)
        out = {"samples": len(self.samples), "seconds": round(self.samples[-1].t - self.samples[0].t, 3),
               "mem_peak_bytes": max(s.mem_used for s in self.samples), "mem_total_bytes": self.samples[-1].mem_total,
               "sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
               "sm_max_mhz": self._max_sm, "power_w": round(statistics.median(pw), 1) if pw else None,
               "reasons": reasons, "rejecting_reasons": [r for r in reasons if r in REJECTING]}
        if self.error:
            out["error"] = self.error
        return out

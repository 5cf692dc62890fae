"""GPU telemetry for the control API: a read-only NVML snapshot cached for one second.

Only queries are issued (name, memory, utilisation, clocks, power, temperature, throttle reasons); nothing here changes
a setting of the GPU.  ``nvml`` can be any object with the ``pynvml`` functions used below, which is how the tests run
without a GPU.  Reference: ``mfq/server/services/hardware.py`` (NVML with a 1 s cache).
"""

from __future__ import annotations

import time


class HardwareMonitor:
    def __init__(self, nvml=None, ttl: float = 1.0, clock=time.monotonic) -> None:
        self.ttl, self.clock = ttl, clock
        self._nvml, self._ready, self._cache, self._stamp = nvml, False, None, -1e9
        self.error: str | None = None

    def _lib(self):
        if self._nvml is None:
            try:
                import pynvml
                self._nvml = pynvml
            except Exception as exc:  # no NVML on this machine
                self.error = f"nvml unavailable: {exc}"
                return None
        if not self._ready:
            try:
                self._nvml.nvmlInit()
                self._ready = True
            except Exception as exc:
                self.error = f"nvmlInit failed: {exc}"
                return None
        return self._nvml

    def snapshot(self) -> dict:
        now = self.clock()
        if self._cache is not None and now - self._stamp < self.ttl:
            return self._cache
        n = self._lib()
        gpus = []
        if n is not None:
            def maybe(fn, *a):
                try:
                    return fn(*a)
                except Exception:
                    return None
            for i in range(n.nvmlDeviceGetCount()):
                h = n.nvmlDeviceGetHandleByIndex(i)
                mem = maybe(n.nvmlDeviceGetMemoryInfo, h)
                util = maybe(n.nvmlDeviceGetUtilizationRates, h)
                name = maybe(n.nvmlDeviceGetName, h)
                power = maybe(n.nvmlDeviceGetPowerUsage, h)
                gpus.append({
                    "index": i, "name": name.decode() if isinstance(name, bytes) else name,
                    "memory_total": getattr(mem, "total", None), "memory_used": getattr(mem, "used", None),
                    "utilization": getattr(util, "gpu", None),
                    "sm_clock_mhz": maybe(n.nvmlDeviceGetClockInfo, h, getattr(n, "NVML_CLOCK_SM", 1)),
                    "power_w": power / 1000.0 if power is not None else None,
                    "temperature_c": maybe(n.nvmlDeviceGetTemperature, h, getattr(n, "NVML_TEMPERATURE_GPU", 0)),
                    "throttle_reasons": maybe(n.nvmlDeviceGetCurrentClocksThrottleReasons, h),
                })
        self._cache = {"gpus": gpus, "error": self.error if n is None else None, "sampled_at": time.time()}
        self._stamp = now
        return self._cache

"""GPU telemetry for the control API: a read-only NVML snapshot cached for one second.

Only queries are issued (name, memory, utilisation, clocks, power, temperature, throttle reasons); nothing here changes
a setting of the GPU.  ``nvml`` can be any object with the ``pynvml`` functions used below, which is how the tests run
without a GPU.  :class:`ResourceHistory` keeps a bounded timeline of those snapshots plus the host's CPU load and memory
(``psutil``), filled by a sampler thread or by explicit :meth:`ResourceHistory.sample` calls.
Reference: ``mfq/server/services/hardware.py`` (NVML with a 1 s cache), ``resource_monitor.py`` (usage timeline).
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


class ResourceHistory:
    """The last ``capacity`` samples of GPU and host usage, one every ``interval`` seconds while the sampler runs."""

    def __init__(self, monitor: HardwareMonitor, capacity: int = 600, interval: float = 1.0, host=None) -> None:
        import collections
        import threading
        self.monitor, self.interval = monitor, interval
        self.samples = collections.deque(maxlen=capacity)
        self._host = host  # an object with cpu_percent() and virtual_memory() (psutil by default)
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._lock = threading.Lock()

    def _host_usage(self) -> dict:
        h = self._host
        if h is None:
            try:
                import psutil
                h = self._host = psutil
            except Exception:
                return {}
        try:
            vm = h.virtual_memory()
            return {"cpu_percent": float(h.cpu_percent(interval=None)), "memory_total": int(vm.total), "memory_used": int(vm.total - vm.available)}
        except Exception:
            return {}

    def sample(self) -> dict:
        snap = self.monitor.snapshot()
        row = {"t": time.time(), "host": self._host_usage(),
               "gpus": [{k: g.get(k) for k in ("index", "memory_used", "utilization", "sm_clock_mhz", "power_w", "temperature_c")}
                        for g in snap.get("gpus", [])]}
        with self._lock:
            self.samples.append(row)
        return row

    def start(self) -> None:
        import threading
        if self._thread is not None:
            return
        self._stop.clear()

        def loop():
            while not self._stop.wait(self.interval):
                self.sample()
        self._thread = threading.Thread(target=loop, name="mfq-resource-history", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
            self._thread = None

    def history(self, last: int | None = None) -> dict:
        with self._lock:
            rows = list(self.samples)
        if last is not None:
            rows = rows[-max(0, int(last)):]
        peak = {}
        for r in rows:
            for g in r["gpus"]:
                p = peak.setdefault(g["index"], {"memory_used": 0, "utilization": 0, "power_w": 0.0})
                for k in p:
                    if g.get(k) is not None:
                        p[k] = max(p[k], g[k])
        return {"interval": self.interval, "capacity": self.samples.maxlen, "samples": rows, "peak": {str(k): v for k, v in peak.items()}}

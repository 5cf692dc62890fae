"""Prometheus text exposition (format 0.0.4) without a client library, with the reference's metric names
(``docs/runtime/metrics.md``; implementation parity ``mfq/server/services/metrics.py``): every series carries
``model`` and ``instance`` labels, request series add ``result``, histograms add ``le``."""

from __future__ import annotations

import threading
from collections import defaultdict

_HELP = {
    "mfq_runtime_batch_capacity": ("gauge", "Rows the loaded model batches together."),
    "mfq_runtime_request_capacity": ("gauge", "Concurrent request slots admitted for this runtime."),
    "mfq_runtime_active_requests": ("gauge", "Requests holding a slot."),
    "mfq_runtime_queued_requests": ("gauge", "Requests waiting for a slot."),
    "mfq_runtime_rejected_requests_total": ("counter", "Requests refused with 429 runtime_queue_full."),
    "mfq_runtime_kv_bytes": ("gauge", "Resident KV bytes."),
    "mfq_runtime_resident_bytes": ("gauge", "Resident memory of the runtime process."),
    "mfq_runtime_kv_usage_ratio": ("gauge", "KV bytes in use over the KV budget."),
    "mfq_runtime_mtp_acceptance_ratio": ("gauge", "Accepted MTP draft tokens over drafted tokens."),
    "mfq_requests_total": ("counter", "Requests served, by result."),
    "mfq_request_prompt_tokens_total": ("counter", "Prompt tokens of served requests."),
    "mfq_request_completion_tokens_total": ("counter", "Completion tokens of served requests."),
    "mfq_request_ttft_seconds": ("histogram", "Time to first token."),
    "mfq_request_prefill_tokens_per_second": ("histogram", "Prefill throughput per request."),
    "mfq_request_decode_tokens_per_second": ("histogram", "Decode throughput per request."),
    "mfq_runtime_queue_wait_seconds": ("histogram", "Time a request waited for a slot."),
}
_BUCKETS = {
    "mfq_request_ttft_seconds": (0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30),
    "mfq_runtime_queue_wait_seconds": (0.001, 0.01, 0.05, 0.1, 0.5, 1, 5, 10, 30),
    "mfq_request_prefill_tokens_per_second": (100, 1000, 5000, 10000, 25000, 50000, 100000, 250000),
    "mfq_request_decode_tokens_per_second": (1, 5, 10, 25, 50, 100, 250, 500, 1000),
}


def _labels(d: dict) -> str:
    def esc(v):
        return str(v).replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n")
    return "{" + ",".join(f'{k}="{esc(v)}"' for k, v in d.items()) + "}"


class Metrics:
    def __init__(self) -> None:
        self._lock = threading.Lock()
        self._counters: dict = defaultdict(float)
        self._hist: dict = {}

    @staticmethod
    def _key(name, model, extra):
        return (name, model.name, model.instance, tuple(sorted(extra.items())))

    def inc(self, name: str, model, by: float = 1.0, **extra) -> None:
        with self._lock:
            self._counters[self._key(name, model, extra)] += by

    def observe(self, name: str, model, value: float, **extra) -> None:
        with self._lock:
            h = self._hist.setdefault(self._key(name, model, extra), {"sum": 0.0, "count": 0, "b": [0] * len(_BUCKETS[name])})
            h["sum"] += value
            h["count"] += 1
            for i, le in enumerate(_BUCKETS[name]):
                if value <= le:
                    h["b"][i] += 1

    def drop_instance(self, model_name: str, instance: str) -> None:
        with self._lock:
            for store in (self._counters, self._hist):
                for k in [k for k in store if k[1] == model_name and k[2] == instance]:
                    del store[k]

    def render(self, service) -> str:
        lines: list[str] = []
        gauges = defaultdict(list)
        for lm in service.models.values():
            base = {"model": lm.name, "instance": lm.instance}
            s = lm.scheduler
            gauges["mfq_runtime_batch_capacity"].append((base, lm.request_capacity))
            gauges["mfq_runtime_request_capacity"].append((base, lm.request_capacity + s.max_queue))
            gauges["mfq_runtime_active_requests"].append((base, len(s.running) + len(s.waiting)))
            gauges["mfq_runtime_queued_requests"].append((base, len(s.waiting)))
            eng = lm.engine
            if hasattr(eng, "cache"):
                used = (eng.cache.num_pages - 1 - eng.cache.allocator.free_pages) * eng.cache.page_size * eng.cache.bytes_per_token()
                total = (eng.cache.num_pages - 1) * eng.cache.page_size * eng.cache.bytes_per_token()
                gauges["mfq_runtime_kv_bytes"].append((base, used))
                gauges["mfq_runtime_kv_usage_ratio"].append((base, used / total if total else 0.0))
            worker = getattr(getattr(s, "worker", None), "proc", None)  # a child runtime: report ITS memory
            rss = _resident_bytes(worker.pid if worker is not None and worker.poll() is None else None)
            if rss:
                gauges["mfq_runtime_resident_bytes"].append((base, rss))
            mtp = getattr(eng, "mtp_stats", None)
            mtp = mtp() if callable(mtp) else mtp
            if mtp and mtp.get("drafted"):
                gauges["mfq_runtime_mtp_acceptance_ratio"].append((base, mtp["accepted"] / mtp["drafted"]))
        for name, rows in gauges.items():
            lines += [f"# HELP {name} {_HELP[name][1]}", f"# TYPE {name} gauge"]
            lines += [f"{name}{_labels(lb)} {val}" for lb, val in rows]
        with self._lock:
            by_name = defaultdict(list)
            for (name, model, inst, extra), v in self._counters.items():
                by_name[name].append(({"model": model, "instance": inst, **dict(extra)}, v))
            for name, rows in by_name.items():
                lines += [f"# HELP {name} {_HELP[name][1]}", f"# TYPE {name} counter"]
                lines += [f"{name}{_labels(lb)} {val:g}" for lb, val in rows]
            hist_by = defaultdict(list)
            for (name, model, inst, extra), h in self._hist.items():
                hist_by[name].append(({"model": model, "instance": inst, **dict(extra)}, h))
            for name, rows in hist_by.items():
                lines += [f"# HELP {name} {_HELP[name][1]}", f"# TYPE {name} histogram"]
                for lb, h in rows:
                    for le, c in zip(_BUCKETS[name], h["b"]):
                        lines.append(f"{name}_bucket{_labels({**lb, 'le': le})} {c}")
                    lines.append(f"{name}_bucket{_labels({**lb, 'le': '+Inf'})} {h['count']}")
                    lines.append(f"{name}_sum{_labels(lb)} {h['sum']:g}")
                    lines.append(f"{name}_count{_labels(lb)} {h['count']}")
        return "\n".join(lines) + "\n"


def _resident_bytes(pid: int | None = None) -> int:
    """Resident set size of this process (or of ``pid``) from ``/proc``; 0 where that is not available."""
    import os
    try:
        with open(f"/proc/{pid or os.getpid()}/statm") as f:
            return int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
    except (OSError, ValueError, IndexError):
        return 0

"""Runtime configuration: one typed record, overridable by ``MFQ_*`` environment variables, validated strictly.

Every default-on optimisation has a kill switch and every tunable a name, as in the reference (its ``MFQ_*`` variables
are parsed once into ``CudaExecutionConfig``, ``cpp_runtime/backends/cuda/ops/cuda_execution.cpp:441-616``, engine-level
ones in ``cpp_runtime/backends/cuda/storage/load_options.cpp:64-95``).  A value that does not parse is an error, not a
silent default: ``MFQ_GEMV=off`` raises instead of leaving the fast path on.

``RuntimeConfig.from_env()`` reads the process environment; :func:`current` caches that record for the code paths that
consult it (``ops.kernels.gemv_enabled``, the engine's defaults, the profiler, the tracer).  ``MFQ_PDL`` and
``MFQ_GEMM_STAGES`` are read by the CUDA library itself at its first launch; they are listed here so that one place
documents and validates all of them.  ``mfq config`` prints the effective record and the table of variables.
"""

from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, fields


def _flag(text: str) -> bool:
    if text not in ("0", "1"):
        raise ValueError("expected 0 or 1")
    return text == "1"


def _stages(text: str) -> int:
    v = int(text)
    if v not in (0, 2, 3, 4, 6, 8):
        raise ValueError("expected 0 (automatic), 2, 3, 4, 6 or 8")
    return v


def _positive(text: str) -> int:
    v = int(text)
    if v <= 0:
        raise ValueError("expected a positive integer")
    return v


def _topics(text: str) -> tuple[str, ...]:
    items = tuple(t for t in text.split(",") if t)
    unknown = [t for t in items if t not in TRACE_TOPICS and t != "all"]
    if unknown:
        raise ValueError(f"unknown trace topic(s) {unknown}; known: {', '.join(TRACE_TOPICS)}")
    return items


TRACE_TOPICS = ("scheduler", "graph", "prefix", "session", "spmd")

# field -> (environment variable, parser, what it does)
_ENV = {
    "gemv": ("MFQ_GEMV", _flag, "weight-streaming FP8 GEMV for <= 16 token rows (0: always the tcgen05 GEMM)"),
    "act_gemv": ("MFQ_ACT_GEMV", _flag, "fold norm / quantization / SwiGLU into the product kernel for <= 4 rows (measured slower: off)"),
    "pdl": ("MFQ_PDL", _flag, "programmatic dependent launch on the decode kernels (read by the CUDA library)"),
    "gemm_stages": ("MFQ_GEMM_STAGES", _stages, "force the TMA ring depth of the FP8 GEMM, 0 = chosen per shape (read by the CUDA library)"),
    "cuda_graphs": ("MFQ_CUDA_GRAPHS", _flag, "capture decode / MTP steps into CUDA graphs (0: eager launches)"),
    "prefill_chunk": ("MFQ_PREFILL_CHUNK", _positive, "longest prompt span prefilled in one pass; longer prompts run in chunks over the cached past"),
    "native_threads": ("MFQ_NATIVE_THREADS", _positive, "worker threads of the host library's decoders and range reads"),
    "profile": ("MFQ_PROFILE", _flag, "named profiling scopes (CUDA events + NVTX + wall clock)"),
    "profile_filter": ("MFQ_PROFILE_FILTER", str, "comma separated name pieces of the scopes to keep"),
    "profile_decode": ("MFQ_PROFILE_DECODE", _flag, "one stderr line per decode call"),
    "trace": ("MFQ_TRACE", _topics, "comma separated trace topics written as key=value lines to stderr: " + ", ".join(TRACE_TOPICS) + " or all"),
}


@dataclass(frozen=True)
class RuntimeConfig:
    gemv: bool = True
    act_gemv: bool = False
    pdl: bool = True
    gemm_stages: int = 0
    cuda_graphs: bool = True
    prefill_chunk: int = 8192
    native_threads: int = 8
    profile: bool = False
    profile_filter: str = ""
    profile_decode: bool = False
    trace: tuple[str, ...] = ()

    @classmethod
    def from_env(cls, env=None) -> "RuntimeConfig":
        env = os.environ if env is None else env
        values = {}
        for f in fields(cls):
            name, parse, _doc = _ENV[f.name]
            if name in env:
                try:
                    values[f.name] = parse(env[name])
                except ValueError as exc:
                    raise ValueError(f"{name}={env[name]!r}: {exc}") from None
        known = {v[0] for v in _ENV.values()}
        stray = sorted(k for k in env if k.startswith("MFQ_") and k not in known and k not in _OTHER)
        if stray:  # a misspelt switch silently does nothing: say so, but do not stop a server over it
            print(f"warning: unknown MFQ_* variable(s) ignored: {', '.join(stray)} (see `mfq config`)", file=sys.stderr)
        return cls(**values)

    def traces(self, topic: str) -> bool:
        return topic in self.trace or "all" in self.trace

    def describe(self) -> list[dict]:
        return [{"variable": _ENV[f.name][0], "value": getattr(self, f.name), "default": f.default, "what": _ENV[f.name][2]}
                for f in fields(self)]


# variables that belong to other parts of the package (launchers, tests), not to this record
_OTHER = {"MFQ_SPMD_PORT"}

_current: RuntimeConfig | None = None


def current() -> RuntimeConfig:
    global _current
    if _current is None:
        _current = RuntimeConfig.from_env()
    return _current


def reload(env=None) -> RuntimeConfig:
    """Re-read the environment (tests; a server reload)."""
    global _current
    _current = RuntimeConfig.from_env(env)
    return _current


def trace(topic: str, event: str, **fields_) -> None:
    """``MFQ_TRACE`` line: ``trace topic=... event=... t=... key=value ...`` on stderr (stdout stays free for frames)."""
    if not current().traces(topic):
        return
    rest = " ".join(f"{k}={v}" for k, v in fields_.items())
    print(f"trace topic={topic} event={event} t={time.monotonic():.6f} {rest}".rstrip(), file=sys.stderr, flush=True)

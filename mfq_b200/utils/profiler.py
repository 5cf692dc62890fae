"""Named profiling scopes: a CUDA-event pair plus the wall clock around any piece of the forward pass.

The counterpart of the reference's ``CudaProfiler::measure(name, fn)`` (``cpp_runtime/backends/cuda/ops/include/
cuda_execution.h:109-158``; report format and name filter in ``ops/cuda_execution.cpp:661-725``): call sites carry
string names (``"attn.qkv"``, ``"ffn.gate_up"``), a filter keeps only the names asked for, and the report is one
``profile_item name=... calls=... cuda_ms=... wall_ms=...`` line per name on stderr.

* Off (the default) a scope is one attribute test and a shared no-op context: nothing is recorded, no event is made.
* On a CUDA device each scope records two timing events on the current stream and opens an NVTX range of the same
  name; elapsed times are read once, in :meth:`Profiler.report` / :meth:`Profiler.items`, after ONE synchronize, so
  profiling adds no host/device synchronisation inside the step.
* While a stream is being captured into a CUDA graph, scopes are skipped (timing events are not capturable); profile
  the eager step (``LLMEngine(use_graphs=False)`` or :func:`profile_engine`) to see the per-op split and time the
  graph replay as a whole with the ``decode.step`` scope.

Environment: ``MFQ_PROFILE=1`` switches the process-wide profiler on, ``MFQ_PROFILE_FILTER=attn,ffn.down`` keeps the
scopes whose name contains one of the comma separated pieces, ``MFQ_PROFILE_DECODE=1`` makes the engine print one
``decode_profile`` line per generated token.
"""

from __future__ import annotations

import contextlib
import os
import sys
import time
from dataclasses import dataclass, field

import torch

_NULL = contextlib.nullcontext()


@dataclass
class ProfileItem:
    name: str
    calls: int = 0
    wall_ms: float = 0.0
    cuda_ms: float = 0.0
    pending: list = field(default_factory=list)  # (start event, end event) pairs not read yet


class _Scope:
    __slots__ = ("prof", "item", "t0", "ev", "nvtx")

    def __init__(self, prof: "Profiler", item: ProfileItem, cuda: bool) -> None:
        self.prof, self.item, self.ev, self.nvtx = prof, item, None, cuda
        self.t0 = 0.0

    def __enter__(self):
        if self.nvtx:
            torch.cuda.nvtx.range_push(self.item.name)
            self.ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self.ev[0].record()
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.item.wall_ms += (time.perf_counter() - self.t0) * 1e3
        self.item.calls += 1
        if self.nvtx:
            self.ev[1].record()
            self.item.pending.append(self.ev)
            torch.cuda.nvtx.range_pop()
        return False


class Profiler:
    def __init__(self, enabled: bool = False, name_filter: str = "") -> None:
        self.enabled = enabled
        self.filter = tuple(p for p in name_filter.split(",") if p)
        self._items: dict[str, ProfileItem] = {}

    @classmethod
    def from_env(cls, env=None) -> "Profiler":
        env = os.environ if env is None else env
        flag = env.get("MFQ_PROFILE", "0")
        if flag not in ("0", "1"):
            raise ValueError(f"MFQ_PROFILE must be 0 or 1, not {flag!r}")
        return cls(flag == "1", env.get("MFQ_PROFILE_FILTER", ""))

    def wants(self, name: str) -> bool:
        return not self.filter or any(p in name for p in self.filter)

    def scope(self, name: str, device=None):
        """Context manager around a piece of work on the current stream of ``device`` (a tensor's device is fine)."""
        if not self.enabled:
            return _NULL
        if not self.wants(name):
            return _NULL
        cuda = device is not None and torch.device(device).type == "cuda"
        if cuda and torch.cuda.is_current_stream_capturing():
            return _NULL
        item = self._items.get(name)
        if item is None:
            item = self._items[name] = ProfileItem(name)
        return _Scope(self, item, cuda)

    def measure(self, name: str, fn, *args, device=None, **kwargs):
        with self.scope(name, device):
            return fn(*args, **kwargs)

    # ---- results -----------------------------------------------------------------------------------------------------
    def items(self) -> list[ProfileItem]:
        """Totals per name in first-use order (synchronizes once if device events are outstanding)."""
        if any(it.pending for it in self._items.values()):
            torch.cuda.synchronize()
        for it in self._items.values():
            for a, b in it.pending:
                it.cuda_ms += a.elapsed_time(b)
            it.pending.clear()
        return list(self._items.values())

    def report(self, file=None) -> list[str]:
        lines = [f"profile_item name={it.name} calls={it.calls} cuda_ms={it.cuda_ms:.3f} wall_ms={it.wall_ms:.3f}"
                 for it in self.items()]
        out = sys.stderr if file is None else file
        for line in lines:
            print(line, file=out)
        return lines

    def reset(self) -> None:
        self._items.clear()


def _from_config() -> Profiler:
    from ..config import current
    cfg = current()
    return Profiler(cfg.profile, cfg.profile_filter)


PROFILER = _from_config()


def scope(name: str, device=None):
    """Scope of the process-wide profiler (what the model and engine code call)."""
    p = PROFILER
    if not p.enabled:
        return _NULL
    return p.scope(name, device)


@contextlib.contextmanager
def profiling(name_filter: str = ""):
    """Switch the process-wide profiler on for a block and hand it out: ``with profiling() as p: ...; p.report()``."""
    p = PROFILER
    saved = (p.enabled, p.filter)
    p.enabled, p.filter = True, tuple(x for x in name_filter.split(",") if x)
    try:
        yield p
    finally:
        p.enabled, p.filter = saved


def profile_engine(engine, prompt_ids, decode_tokens: int = 8, name_filter: str = "") -> list[ProfileItem]:
    """Per-op split of one prefill and ``decode_tokens`` EAGER decode steps of row 0 (graphs are bypassed so that every
    scope inside the forward pass is timed; the kernels are the ones the graph replays)."""
    saved = engine.use_graphs
    engine.use_graphs = False
    PROFILER.reset()
    try:
        with profiling(name_filter) as p:
            engine.prefill(0, prompt_ids)
            for _ in range(decode_tokens):
                engine.decode([0])
            return p.items()
    finally:
        engine.use_graphs = saved
        engine.release(0)

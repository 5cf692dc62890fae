"""Host-side rank health for multi-GPU serving: heartbeats, failure reports, and re-forming the group.

Kernels never wait unboundedly on a peer (every device-side wait has a time budget and reports through a status
word), but a step whose peer died would still burn that budget on every launch.  So ranks talk on the HOST between
steps, through the ``torch.distributed`` key-value store they already share:

* ``beat()`` after every step bumps this rank's counter and timestamp;
* ``report_failure(reason)`` (called from an ``except`` around the step, or after ``Workspace.check()`` found a
  timed-out wait) marks the rank as failed before the process leaves;
* ``check()`` before the next launch raises :class:`RankFailure` naming the ranks that reported a failure or whose
  heartbeat is older than ``timeout`` seconds;
* ``survivors()`` / :func:`reform_group` build the new, smaller process group (the caller then reloads weight shards
  for the new world size -- tensor-parallel shards are cut per world size at load time).

A rank only ever leaves BETWEEN steps, with none of its kernels or collectives in flight.  The reference detects a
dead runtime on the host as well (worker ``poll()``, health latch, revive with back-off:
``mfq/server/runtime/runtime_pool.py:3394-3426``, ``cpp_runtime/scheduler/scheduler.cpp:373-392``).
"""

from __future__ import annotations

import time
from typing import Callable

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, failed: dict[int, str]) -> None:
        super().__init__("rank(s) " + ", ".join(f"{r} ({why})" for r, why in sorted(failed.items())) + " left the group")
        self.failed = failed


class RankHealth:
    def __init__(self, store, rank: int, world: int, *, timeout: float = 10.0, prefix: str = "health",
                 clock: Callable[[], float] = time.time) -> None:
        self.store, self.rank, self.world, self.timeout, self.prefix, self.clock = store, rank, world, timeout, prefix, clock
        self.step = 0
        self.beat()

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self) -> None:
        self.step += 1
        self.store.set(self._key("beat", self.rank), f"{self.step}:{self.clock():.6f}")

    def report_failure(self, reason: str) -> None:
        self.store.set(self._key("failed", self.rank), reason[:200] or "failed")

    def _get(self, key: str) -> str | None:
        # check() must not block on a key a dead rank never wrote: query existence first
        if not self.store.check([key]):
            return None
        return self.store.get(key).decode()

    def failed(self) -> dict[int, str]:
        out: dict[int, str] = {}
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            why = self._get(self._key("failed", r))
            if why is not None:
                out[r] = why
                continue
            beat = self._get(self._key("beat", r))
            if beat is None:
                out[r] = "never joined"
            elif now - float(beat.split(":")[1]) > self.timeout:
                out[r] = f"no heartbeat for {now - float(beat.split(':')[1]):.1f} s"
        return out

    def check(self) -> None:
        bad = self.failed()
        if bad:
            raise RankFailure(bad)

    def survivors(self) -> list[int]:
        bad = self.failed()
        return [r for r in range(self.world) if r not in bad]


def reform_group(survivors: list[int], backend: str | None = None, timeout_s: float = 30.0):
    """New process group of the surviving ranks (every survivor must call this with the same list).  Returns
    ``(group, new_rank, new_world)``."""
    import datetime
    group = dist.new_group(ranks=survivors, backend=backend, timeout=datetime.timedelta(seconds=timeout_s))
    me = dist.get_rank()
    return group, survivors.index(me), len(survivors)

"""Multi-model runtime pool: LRU residency of engine instances and a per-instance priority slot gate.

* at most ``max_instances`` models are resident; loading another evicts the least recently used idle one (a model with
  requests in flight is never evicted); idle models past ``idle_ttl`` are dropped by :meth:`RuntimePool.reap`;
* every instance admits ``concurrency`` requests at once; the rest wait in a bounded priority queue (higher priority
  first, then arrival).  A full queue answers ``runtime_queue_full`` (429), a wait longer than ``queue_timeout``
  ``runtime_queue_timeout`` (503), a passed deadline ``runtime_deadline_exceeded`` (504).

Reference: ``mfq/server/runtime/runtime_pool.py:196-252,415,669`` (pool, slot gate, budgets).  The clock is injectable
so that the tests need no sleeping.
"""

from __future__ import annotations

import heapq
import itertools
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable

from ..engine.scheduler import DeadlineExceeded, QueueFull, QueueTimeout


class SlotGate:
    """``concurrency`` slots + bounded priority queue.  ``acquire`` blocks until a slot is free or fails."""

    def __init__(self, concurrency: int, max_queue: int = 64, clock: Callable[[], float] = time.monotonic) -> None:
        self.concurrency, self.max_queue, self.clock = concurrency, max_queue, clock
        self._cv = threading.Condition()
        self._active = 0
        self._waiting: list[tuple[int, int, object]] = []  # (-priority, ticket, token)
        self._tickets = itertools.count()
        self.stats = {"admitted": 0, "rejected_full": 0, "timeouts": 0, "deadline": 0}

    @property
    def active(self) -> int:
        return self._active

    @property
    def queued(self) -> int:
        return len(self._waiting)

    def try_acquire(self) -> bool:
        with self._cv:
            if self._active < self.concurrency and not self._waiting:
                self._active += 1
                self.stats["admitted"] += 1
                return True
            return False

    def acquire(self, priority: int = 0, queue_timeout: float | None = None, deadline: float | None = None,
                wait: Callable[[threading.Condition, float | None], None] | None = None) -> None:
        """Blocks.  ``wait(cv, seconds)`` may be supplied by tests to advance a fake clock instead of sleeping."""
        with self._cv:
            if self._active < self.concurrency and not self._waiting:
                self._active += 1
                self.stats["admitted"] += 1
                return
            if len(self._waiting) >= self.max_queue:
                self.stats["rejected_full"] += 1
                raise QueueFull(f"{len(self._waiting)} requests already wait for this model")
            token = object()
            entry = (-priority, next(self._tickets), token)
            heapq.heappush(self._waiting, entry)
            start = self.clock()
            try:
                while True:
                    now = self.clock()
                    if deadline is not None and now >= deadline:
                        self.stats["deadline"] += 1
                        raise DeadlineExceeded("deadline passed while waiting for a slot")
                    if queue_timeout is not None and now - start >= queue_timeout:
                        self.stats["timeouts"] += 1
                        raise QueueTimeout("waited too long for a slot")
                    if self._active < self.concurrency and self._waiting[0][2] is token:
                        heapq.heappop(self._waiting)
                        self._active += 1
                        self.stats["admitted"] += 1
                        self._cv.notify_all()
                        return
                    limits = [x for x in ((deadline - now) if deadline is not None else None,
                                          (queue_timeout - (now - start)) if queue_timeout is not None else None) if x is not None]
                    (wait or (lambda cv, s: cv.wait(s)))(self._cv, min(limits) if limits else None)
            except BaseException:
                if entry in self._waiting:
                    self._waiting.remove(entry)
                    heapq.heapify(self._waiting)
                    self._cv.notify_all()
                raise

    def release(self) -> None:
        with self._cv:
            self._active = max(0, self._active - 1)
            self._cv.notify_all()


@dataclass
class Instance:
    name: str
    runtime: Any
    gate: SlotGate
    last_used: float
    loads: int = 1
    meta: dict = field(default_factory=dict)


class RuntimePool:
    def __init__(self, loader: Callable[[str], Any], *, max_instances: int = 1, concurrency: int = 32, max_queue: int = 64,
                 idle_ttl: float | None = None, unloader: Callable[[Any], None] | None = None,
                 clock: Callable[[], float] = time.monotonic) -> None:
        self.loader, self.unloader = loader, unloader
        self.max_instances, self.concurrency, self.max_queue, self.idle_ttl, self.clock = max_instances, concurrency, max_queue, idle_ttl, clock
        self._lock = threading.RLock()
        self.instances: dict[str, Instance] = {}
        self.evictions = 0

    def _drop(self, name: str) -> None:
        inst = self.instances.pop(name)
        if self.unloader:
            self.unloader(inst.runtime)
        self.evictions += 1

    def get(self, name: str) -> Instance:
        """Resident instance of ``name`` (loading it, and evicting the least recently used idle model, if needed)."""
        with self._lock:
            inst = self.instances.get(name)
            if inst is None:
                while len(self.instances) >= self.max_instances:
                    idle = [i for i in self.instances.values() if i.gate.active == 0 and i.gate.queued == 0]
                    if not idle:
                        raise QueueFull("every resident model is busy; cannot load another")
                    self._drop(min(idle, key=lambda i: i.last_used).name)
                inst = Instance(name, self.loader(name), SlotGate(self.concurrency, self.max_queue, self.clock), self.clock())
                self.instances[name] = inst
            inst.last_used = self.clock()
            return inst

    def unload(self, name: str) -> bool:
        with self._lock:
            inst = self.instances.get(name)
            if inst is None or inst.gate.active or inst.gate.queued:
                return False
            self._drop(name)
            return True

    def reap(self) -> list[str]:
        """Drop idle instances older than ``idle_ttl``; returns their names."""
        if self.idle_ttl is None:
            return []
        with self._lock:
            now = self.clock()
            old = [i.name for i in self.instances.values() if i.gate.active == 0 and i.gate.queued == 0 and now - i.last_used > self.idle_ttl]
            for name in old:
                self._drop(name)
            return old

    def snapshot(self) -> dict:
        with self._lock:
            return {"max_instances": self.max_instances, "evictions": self.evictions,
                    "instances": [{"name": i.name, "active": i.gate.active, "queued": i.gate.queued, "concurrency": i.gate.concurrency,
                                   "idle_seconds": self.clock() - i.last_used, **i.gate.stats} for i in self.instances.values()]}

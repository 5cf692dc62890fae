"""Multi-model runtime pool: LRU residency of engine instances and a per-instance priority slot gate.

* at most ``max_instances`` models are resident; loading another evicts the least recently used idle one (a model with
  requests in flight is never evicted); idle models past ``idle_ttl`` are dropped by :meth:`RuntimePool.reap`;
* with ``max_memory_bytes`` the pool also budgets device memory: an instance declares its weight bytes (``sizer``),
  loading evicts idle models least-recently-used first until the newcomer fits, and :meth:`RuntimePool.rebalance` splits
  what the weights leave among the resident models as their KV budgets (by ``kv_share``), telling each runtime through
  ``set_kv_budget`` when it has one; a loader failure is remembered for ``load_failure_cooldown`` seconds, so a broken
  artifact is not re-opened on every request;
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
    weight_bytes: int = 0
    kv_budget_bytes: int = 0
    kv_share: float = 1.0
    idle_ttl: float | None = None  # overrides the pool's


class RuntimePool:
    def __init__(self, loader: Callable[[str], Any], *, max_instances: int = 1, concurrency: int = 32, max_queue: int = 64,
                 idle_ttl: float | None = None, unloader: Callable[[Any], None] | None = None,
                 clock: Callable[[], float] = time.monotonic, max_memory_bytes: int | None = None,
                 sizer: Callable[[str], int] | None = None, min_kv_bytes: int = 0, load_failure_cooldown: float = 30.0) -> None:
        self.loader, self.unloader = loader, unloader
        self.max_memory_bytes, self.sizer, self.min_kv_bytes = max_memory_bytes, sizer, min_kv_bytes
        self.load_failure_cooldown = load_failure_cooldown
        self._failures: dict[str, tuple[float, BaseException]] = {}
        self.max_instances, self.concurrency, self.max_queue, self.idle_ttl, self.clock = max_instances, concurrency, max_queue, idle_ttl, clock
        self._lock = threading.RLock()
        self.instances: dict[str, Instance] = {}
        self.evictions = 0

    def _drop(self, name: str) -> None:
        inst = self.instances.pop(name)
        if self.unloader:
            self.unloader(inst.runtime)
        self.evictions += 1
        self.rebalance()

    def get(self, name: str) -> Instance:
        """Resident instance of ``name`` (loading it, and evicting the least recently used idle model, if needed)."""
        with self._lock:
            inst = self.instances.get(name)
            if inst is None:
                failed = self._failures.get(name)
                if failed is not None:
                    if self.clock() - failed[0] < self.load_failure_cooldown:
                        raise failed[1]
                    del self._failures[name]
                need = int(self.sizer(name)) if self.sizer else 0

                def evict_one(why: str) -> None:
                    idle = [i for i in self.instances.values() if i.gate.active == 0 and i.gate.queued == 0]
                    if not idle:
                        raise QueueFull(why)
                    self._drop(min(idle, key=lambda i: i.last_used).name)
                while len(self.instances) >= self.max_instances:
                    evict_one("every resident model is busy; cannot load another")
                if self.max_memory_bytes is not None:
                    if need + self.min_kv_bytes > self.max_memory_bytes:
                        raise MemoryError(f"{name} needs {need + self.min_kv_bytes} bytes, the runtime budget is {self.max_memory_bytes}")
                    while self._weights() + need + self.min_kv_bytes * (len(self.instances) + 1) > self.max_memory_bytes:
                        evict_one("resident models are busy and leave no memory for another")
                try:
                    runtime = self.loader(name)
                except BaseException as exc:
                    self._failures[name] = (self.clock(), exc)
                    raise
                inst = Instance(name, runtime, SlotGate(self.concurrency, self.max_queue, self.clock), self.clock(), weight_bytes=need)
                self.instances[name] = inst
                self.rebalance()
            inst.last_used = self.clock()
            return inst

    def _weights(self) -> int:
        return sum(i.weight_bytes for i in self.instances.values())

    def rebalance(self) -> dict[str, int]:
        """Split the memory the weights leave among the resident models' KV caches in proportion to ``kv_share``
        (never below ``min_kv_bytes``); runtimes that expose ``set_kv_budget(bytes)`` are told.  Returns the budgets."""
        with self._lock:
            if self.max_memory_bytes is None or not self.instances:
                return {}
            free = max(0, self.max_memory_bytes - self._weights())
            total = sum(max(i.kv_share, 0.0) for i in self.instances.values()) or 1.0
            out = {}
            for i in self.instances.values():
                budget = max(self.min_kv_bytes, int(free * max(i.kv_share, 0.0) / total))
                if budget != i.kv_budget_bytes:
                    i.kv_budget_bytes = budget
                    setter = getattr(i.runtime, "set_kv_budget", None)
                    if callable(setter):
                        setter(budget)
                out[i.name] = budget
            return out

    def configure(self, name: str, *, kv_share: float | None = None, idle_ttl: float | None = ...) -> None:
        """Per-model settings of a resident instance (a policy change applies at once)."""
        with self._lock:
            inst = self.instances[name]
            if kv_share is not None:
                inst.kv_share = float(kv_share)
            if idle_ttl is not ...:
                inst.idle_ttl = idle_ttl
            self.rebalance()

    def unload(self, name: str) -> bool:
        with self._lock:
            inst = self.instances.get(name)
            if inst is None or inst.gate.active or inst.gate.queued:
                return False
            self._drop(name)
            return True

    def reap(self) -> list[str]:
        """Drop idle instances older than ``idle_ttl``; returns their names."""
        with self._lock:
            now = self.clock()

            def ttl(i):
                return i.idle_ttl if i.idle_ttl is not None else self.idle_ttl
            old = [i.name for i in self.instances.values()
                   if ttl(i) is not None and i.gate.active == 0 and i.gate.queued == 0 and now - i.last_used > ttl(i)]
            for name in old:
                self._drop(name)
            return old

    def snapshot(self) -> dict:
        with self._lock:
            return {"max_instances": self.max_instances, "evictions": self.evictions,
                    "instances": [{"name": i.name, "active": i.gate.active, "queued": i.gate.queued, "concurrency": i.gate.concurrency,
                                   "idle_seconds": self.clock() - i.last_used, "weight_bytes": i.weight_bytes,
                                   "kv_budget_bytes": i.kv_budget_bytes, **i.gate.stats} for i in self.instances.values()],
                    "max_memory_bytes": self.max_memory_bytes, "weight_bytes": self._weights()}

"""Model service: owns one engine + scheduler per loaded model and runs them on a worker thread.

HTTP handlers submit :class:`~mfq_b200.engine.scheduler.Request` objects and consume per-request event queues;
the worker thread is the only one that touches the GPU (the reference keeps the same discipline with a single
scheduler thread that owns the engine, ``cpp_runtime/scheduler/scheduler.cpp:236``).  A small LRU pool bounds the
number of resident models (``--max-runtime-instances`` in the reference's ``RuntimePool``).
"""

from __future__ import annotations

import queue
import threading
import time
import uuid
from collections import OrderedDict
from dataclasses import dataclass, field

from ..engine.scheduler import (BackendFailure, ContinuousBatchScheduler, Event, QueueFull, Request, SamplingParams)
from .metrics import Metrics


@dataclass
class LoadedModel:
    name: str
    engine: object
    tokenizer: object
    scheduler: ContinuousBatchScheduler
    instance: str = field(default_factory=lambda: str(uuid.uuid4()))
    loaded_at: float = field(default_factory=time.time)
    request_capacity: int = 0
    meta: dict = field(default_factory=dict)  # header_extra / assets / architecture of the checkpoint, when known


class ModelService:
    def __init__(self, *, max_instances: int = 1, max_queue: int = 256, queue_timeout: float | None = 30.0,
                 loader=None, idle_timeout: float | None = None) -> None:
        self.idle_timeout = idle_timeout  # unload a model nobody used for this long (it loads again on demand)
        self.models: OrderedDict[str, LoadedModel] = OrderedDict()
        self.max_instances, self.max_queue, self.queue_timeout = max_instances, max_queue, queue_timeout
        self.metrics = Metrics()
        self.loader = loader  # callable(name) -> (engine, tokenizer), for /api/v1/models/load
        self._inbox: queue.Queue = queue.Queue()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, name="mfq-engine", daemon=True)
        self._thread.start()

    # ---- model pool ----------------------------------------------------------------------------------------------
    def add_model(self, name: str, engine, tokenizer) -> LoadedModel:
        while len(self.models) >= self.max_instances and name not in self.models:
            victim, _ = next(iter(self.models.items()))
            self.unload(victim)
        sched = ContinuousBatchScheduler(engine, max_queue=self.max_queue, queue_timeout=self.queue_timeout)
        lm = LoadedModel(name, engine, tokenizer, sched, request_capacity=getattr(engine, "max_batch", 1))
        about = getattr(engine, "checkpoint_meta", None) or getattr(getattr(engine, "engine", None), "checkpoint_meta", None)
        if about:
            lm.meta.update(about)
        self.models[name] = lm
        return lm

    def add_worker_model(self, name: str, command: list[str], tokenizer, *, capacity: int = 32, env: dict | None = None,
                         **worker_kw) -> LoadedModel:
        """A model that runs in a child runtime process (see ``server/worker.py``): the child owns the engine, this
        process keeps the tokenizer, the queue limits and the watch over the child."""
        from .worker import WorkerScheduler
        while len(self.models) >= self.max_instances and name not in self.models:
            victim, _ = next(iter(self.models.items()))
            self.unload(victim)
        sched = WorkerScheduler(command, capacity=capacity, max_queue=self.max_queue, env=env, **worker_kw)
        lm = LoadedModel(name, None, tokenizer, sched, request_capacity=capacity, meta={"worker": True})
        self.models[name] = lm
        return lm

    def load(self, name: str) -> LoadedModel:
        if name in self.models:
            self.models.move_to_end(name)
            return self.models[name]
        if self.loader is None:
            raise KeyError(name)
        engine, tok = self.loader(name)
        return self.add_model(name, engine, tok)

    def unload(self, name: str) -> bool:
        lm = self.models.pop(name, None)
        if lm is None:
            return False
        if hasattr(lm.scheduler, "shutdown"):  # a worker process: end the child with the model
            lm.scheduler.shutdown()
        self.metrics.drop_instance(lm.name, lm.instance)
        return True

    def resolve(self, name: str | None) -> LoadedModel:
        if name and name in self.models:
            self.models.move_to_end(name)
            return self.models[name]
        if name and self.loader is not None:
            return self.load(name)
        if not self.models:
            raise KeyError(name or "<none loaded>")
        if name:
            raise KeyError(name)
        return next(reversed(self.models.values()))

    # ---- requests ------------------------------------------------------------------------------------------------
    def submit(self, model: LoadedModel, prompt_ids: list[int], params: SamplingParams, *, priority: int = 0,
               timeout_seconds: float | None = None, session: str | None = None) -> tuple[Request, "queue.Queue[Event]"]:
        events: "queue.Queue[Event]" = queue.Queue()
        model.meta["last_used"] = time.monotonic()
        req = Request(prompt_ids, params, priority=priority, timeout_seconds=timeout_seconds, on_event=events.put,
                      session=str(session) if session else None)
        done = threading.Event()
        box: dict = {}
        self._inbox.put(("submit", model, req, box, done))
        done.wait()
        if "error" in box:
            if isinstance(box["error"], QueueFull):
                self.metrics.inc("mfq_runtime_rejected_requests_total", model)
            raise box["error"]
        return req, events

    def call(self, model: LoadedModel, fn, timeout: float = 120.0):
        """Run ``fn(model)`` on the serving thread, between scheduling steps (engine state has one owner), and return
        its result or raise what it raised."""
        box: dict = {}
        done = threading.Event()
        self._inbox.put(("call", model, fn, box, done))
        if not done.wait(timeout):
            raise TimeoutError("the serving thread did not get to the call in time")
        if "error" in box:
            raise box["error"]
        return box.get("result")

    def cancel(self, model: LoadedModel, request_id: int) -> None:
        self._inbox.put(("cancel", model, request_id, None, None))

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                while True:
                    kind, model, arg, box, done = self._inbox.get_nowait()
                    if kind == "submit":
                        try:
                            model.scheduler.submit(arg)
                        except Exception as exc:
                            box["error"] = exc
                        done.set()
                    elif kind == "cancel":
                        model.scheduler.cancel(arg)
                    elif kind == "call":
                        try:
                            box["result"] = arg(model)
                        except Exception as exc:
                            box["error"] = exc
                        done.set()
            except queue.Empty:
                pass
            busy = False
            for lm in list(self.models.values()):
                if not lm.scheduler.idle and lm.scheduler.healthy:
                    try:
                        busy |= lm.scheduler.step()
                    except Exception:  # scheduler bug: poison this model only
                        lm.scheduler.healthy = False
            if not busy:
                self._reap_idle()
                time.sleep(0.002)

    def _reap_idle(self) -> None:
        """Unload models that finished their work ``idle_timeout`` seconds ago; only when a loader can bring them back."""
        if not self.idle_timeout or self.loader is None:
            return
        now = time.monotonic()
        for name, lm in list(self.models.items()):
            last = lm.meta.get("last_used", lm.meta.setdefault("last_used", now))
            if lm.scheduler.idle and now - last > self.idle_timeout:
                self.unload(name)

    def shutdown(self) -> None:
        self._stop.set()
        self._thread.join(timeout=5)
        for lm in self.models.values():
            if hasattr(lm.scheduler, "shutdown"):
                lm.scheduler.shutdown()

    # ---- observation ---------------------------------------------------------------------------------------------
    def record_completion(self, model: LoadedModel, req: Request, result: str) -> None:
        m = self.metrics
        m.inc("mfq_requests_total", model, result=result)
        m.inc("mfq_request_prompt_tokens_total", model, by=len(req.prompt))
        m.inc("mfq_request_completion_tokens_total", model, by=len(req.generated))
        if req.first_token_time is not None:
            m.observe("mfq_request_ttft_seconds", model, req.first_token_time - req.arrival)
            dt = time.monotonic() - req.first_token_time
            if len(req.generated) > 1 and dt > 0:
                m.observe("mfq_request_decode_tokens_per_second", model, (len(req.generated) - 1) / dt)

    def status(self) -> dict:
        out = []
        for lm in self.models.values():
            s = lm.scheduler
            extra = {"worker_restarts": s.restarts, "worker_failures": s.failures} if hasattr(s, "restarts") else {}
            out.append({**extra, "model": lm.name, "instance": lm.instance, "healthy": s.healthy, "running": len(s.running),
                        "queued": len(s.waiting), "batch_capacity": lm.request_capacity, "stats": vars(s.stats),
                        "kv_free_tokens": lm.engine.free_tokens() if hasattr(lm.engine, "free_tokens") else None})
        return {"instances": out}

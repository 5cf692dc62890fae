"""Continuous batching: admission, prefill/decode alternation, retraction, deadlines, failure isolation.

Semantics follow the reference engine so that clients see the same behaviour:

* requests wait in a bounded priority queue (full -> ``runtime_queue_full``; waiting past the queue timeout ->
  ``runtime_queue_timeout``; a request past its deadline -> ``runtime_deadline_exceeded``), stable by priority
  then arrival (``cpp_runtime/scheduler/scheduler.cpp:236-421``);
* a request is admitted only if its KV reservation fits: prompt tokens + ``ratio x max_new_tokens`` for it and for
  the already running rows, where the new-token ratio decays from 0.7 to 0.098 over 600 decode steps -- optimistic
  packing that relies on retraction (``cpp_runtime/engine/include/kv_admission.h:12-55``);
* when decode cannot grow every row's KV, rows are retracted -- fewest produced tokens first, longest prompt
  breaking ties -- their pages are freed and they re-enter the queue with prompt + generated tokens
  (``continuous_batch.h:103-125``);
* prefill and decode alternate; a failure inside one request's prefill fails only that request; a failure of the
  batched decode marks the backend unhealthy and fails every request with ``backend_failure``
  (``request_executor.h:127-133``).

The scheduler drives a *backend* with four methods (``prefill``, ``decode``, ``release``, capacity queries), which the
GPU engine and the test doubles implement; it owns no GPU state itself.
"""

from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Callable, Protocol

from ..config import trace

INITIAL_NEW_TOKEN_RATIO = 0.7
MIN_NEW_TOKEN_RATIO = 0.098
RATIO_DECAY_STEPS = 600


class QueueFull(Exception):
    code, status = "runtime_queue_full", 429


class QueueTimeout(Exception):
    code, status = "runtime_queue_timeout", 503


class DeadlineExceeded(Exception):
    code, status = "runtime_deadline_exceeded", 504


class BackendFailure(Exception):
    code, status = "backend_failure", 500


@dataclass
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0
    stop_token_ids: tuple[int, ...] = ()
    enable_mtp: bool = False
    mtp_max_draft_tokens: int = 3
    logit_bias: dict | None = None  # token id -> additive bias in [-100, 100] (OpenAI semantics)
    response_format: dict | str | None = None  # {"type": "json_object"}: constrain the output to a JSON document


@dataclass
class Request:
    prompt: list[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    priority: int = 0
    timeout_seconds: float | None = None
    on_event: Callable[["Event"], None] | None = None
    session: str | None = None  # conversation id: the backend may keep / restore a snapshot of its KV state
    id: int = -1
    # runtime state
    arrival: float = 0.0
    deadline: float | None = None
    generated: list[int] = field(default_factory=list)
    row: int = -1
    first_token_time: float | None = None
    start_time: float | None = None
    retractions: int = 0
    finished: bool = False
    finish_reason: str | None = None
    error: Exception | None = None

    @property
    def context(self) -> list[int]:
        """Tokens to prefill when (re)admitted: the prompt plus anything generated before a retraction."""
        return self.prompt + self.generated


@dataclass
class Event:
    kind: str  # "token" | "completed" | "failed" | "retracted"
    request_id: int
    token: int | None = None
    finish_reason: str | None = None
    error_code: str | None = None
    metrics: dict | None = None


class Backend(Protocol):
    max_batch: int

    def free_tokens(self) -> int: ...
    def tokens_needed(self, tokens: int) -> int: ...
    def prefill(self, row: int, tokens: list[int], params: SamplingParams) -> int: ...
    def decode(self, rows: list[int]) -> dict[int, int | list[int]]: ...  # a list: tokens confirmed by one MTP cycle
    def can_grow(self, row: int) -> bool: ...
    def release(self, row: int) -> None: ...


@dataclass
class SchedulerStats:
    admitted: int = 0
    completed: int = 0
    failed: int = 0
    retractions: int = 0
    decode_steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    queue_rejections: int = 0


class ContinuousBatchScheduler:
    def __init__(self, backend: Backend, *, max_queue: int = 256, queue_timeout: float | None = None,
                 clock: Callable[[], float] = time.monotonic) -> None:
        self.backend = backend
        self.max_queue, self.queue_timeout, self.clock = max_queue, queue_timeout, clock
        self.waiting: list[Request] = []
        self.running: dict[int, Request] = {}  # row -> request
        self.healthy = True
        self.stats = SchedulerStats()
        self.new_token_ratio = INITIAL_NEW_TOKEN_RATIO
        self._ids = itertools.count(1)
        self._decode_next = False

    # ---- client side --------------------------------------------------------------------------------------------
    def submit(self, req: Request) -> int:
        if not self.healthy:
            raise BackendFailure("engine is unhealthy")
        if len(self.waiting) >= self.max_queue:
            self.stats.queue_rejections += 1
            raise QueueFull(f"queue holds {len(self.waiting)} requests")
        req.id = next(self._ids)
        req.arrival = self.clock()
        req.deadline = req.arrival + req.timeout_seconds if req.timeout_seconds else None
        self.waiting.append(req)
        self.waiting.sort(key=lambda r: (-r.priority, r.arrival, r.id))  # stable: priority, then arrival
        return req.id

    def cancel(self, request_id: int) -> bool:
        for r in list(self.waiting):
            if r.id == request_id:
                self.waiting.remove(r)
                self._finish(r, "cancelled")
                return True
        for row, r in list(self.running.items()):
            if r.id == request_id:
                self._release(row)
                self._finish(r, "cancelled")
                return True
        return False

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- internals ----------------------------------------------------------------------------------------------
    def _emit(self, req: Request, ev: Event) -> None:
        if req.on_event:
            req.on_event(ev)

    def _metrics(self, req: Request) -> dict:
        now = self.clock()
        return {"prompt_tokens": len(req.prompt), "completion_tokens": len(req.generated),
                "ttft_s": (req.first_token_time - req.arrival) if req.first_token_time else None,
                "total_s": now - req.arrival, "retractions": req.retractions}

    def _finish(self, req: Request, reason: str) -> None:
        req.finished, req.finish_reason = True, reason
        self.stats.completed += 1
        trace("scheduler", "finish", request=req.id, reason=reason, generated=len(req.generated), retractions=req.retractions)
        self._emit(req, Event("completed", req.id, finish_reason=reason, metrics=self._metrics(req)))

    def _fail(self, req: Request, exc: Exception) -> None:
        req.finished, req.error = True, exc
        req.finish_reason = getattr(exc, "code", "error")
        self.stats.failed += 1
        trace("scheduler", "fail", request=req.id, code=req.finish_reason)
        self._emit(req, Event("failed", req.id, error_code=req.finish_reason, metrics=self._metrics(req)))

    def _snapshot(self, req: Request) -> None:
        """A finished turn of a conversation leaves its KV state with the backend for the next turn."""
        if req.session is not None and hasattr(self.backend, "save_session"):
            try:
                self.backend.save_session(req.row, req.session, req.context)
            except Exception:  # a snapshot is an optimisation: never fail the request over it
                pass

    def _release(self, row: int) -> None:
        self.running.pop(row, None)
        self.backend.release(row)

    def _free_row(self) -> int | None:
        for row in range(self.backend.max_batch):
            if row not in self.running:
                return row
        return None

    def _reserved_tokens(self) -> int:
        """Expected further growth of the running rows under the current new-token ratio."""
        total = 0
        for r in self.running.values():
            remaining = max(0, r.params.max_tokens - len(r.generated))
            total += self.backend.tokens_needed(int(remaining * self.new_token_ratio))
        return total

    def can_admit(self, req: Request) -> bool:
        need = self.backend.tokens_needed(len(req.context) + int(req.params.max_tokens * self.new_token_ratio))
        return need + self._reserved_tokens() <= self.backend.free_tokens()

    def _expire(self) -> None:
        now = self.clock()
        for r in list(self.waiting):
            if r.deadline is not None and now > r.deadline:
                self.waiting.remove(r)
                self._fail(r, DeadlineExceeded("deadline passed while queued"))
            elif self.queue_timeout is not None and r.retractions == 0 and now - r.arrival > self.queue_timeout:
                self.waiting.remove(r)
                self._fail(r, QueueTimeout("waited too long for a slot"))
        for row, r in list(self.running.items()):
            if r.deadline is not None and now > r.deadline:
                self._release(row)
                self._fail(r, DeadlineExceeded("deadline passed during generation"))

    def _accept_token(self, req: Request, tok: int) -> bool:
        """Record a generated token; returns True when the request is done."""
        if req.first_token_time is None:
            req.first_token_time = self.clock()
        req.generated.append(tok)
        self._emit(req, Event("token", req.id, token=tok))
        if tok in req.params.stop_token_ids:
            req.finish_reason = "stop"
            return True
        if len(req.generated) >= req.params.max_tokens:
            req.finish_reason = "length"
            return True
        return False

    def _retract_one(self) -> bool:
        """Free the pages of the row that loses least: fewest produced tokens, longest prompt breaking ties."""
        if not self.running:
            return False
        row, victim = min(self.running.items(), key=lambda kv: (len(kv[1].generated), -len(kv[1].prompt)))
        self._release(row)
        victim.row = -1
        victim.retractions += 1
        self.stats.retractions += 1
        trace("scheduler", "retract", request=victim.id, row=row, generated=len(victim.generated))
        self.new_token_ratio = min(INITIAL_NEW_TOKEN_RATIO, self.new_token_ratio + 0.1)  # be less optimistic for a while
        self._emit(victim, Event("retracted", victim.id))
        self.waiting.insert(0, victim)
        self.waiting.sort(key=lambda r: (-r.priority, r.arrival, r.id))
        return True

    # ---- one scheduling step ------------------------------------------------------------------------------------
    def _try_prefill(self) -> bool:
        for req in self.waiting:
            row = self._free_row()
            if row is None or not self.can_admit(req):
                # a request that can never fit must not block the queue forever
                if row is not None and not self.running and not self.can_admit(req):
                    self.waiting.remove(req)
                    self._fail(req, QueueFull("request needs more KV memory than the engine has"))
                    return True
                return False
            self.waiting.remove(req)
            req.row, req.start_time = row, self.clock()
            self.running[row] = req
            self.stats.admitted += 1
            trace("scheduler", "admit", request=req.id, row=row, context=len(req.context), waiting=len(self.waiting),
                  running=len(self.running), replay=int(bool(req.generated)))
            try:
                extra = {}
                if req.session is not None and hasattr(self.backend, "save_session"):
                    extra["session"] = req.session
                if req.generated and (req.params.response_format or req.params.logit_bias):  # replay after a retraction: the grammar has to
                    extra["generated"] = len(req.generated)       # re-read what was generated before
                tok = self.backend.prefill(row, req.context, req.params, **extra)
            except MemoryError:
                self.running.pop(row, None)
                self.backend.release(row)
                req.row = -1
                self.waiting.insert(0, req)
                return False
            except Exception as exc:  # isolate: only this request fails
                self.running.pop(row, None)
                self.backend.release(row)
                self._fail(req, exc)
                return True
            self.stats.prefill_tokens += len(req.context)
            if self._accept_token(req, tok):
                self._snapshot(req)
                self._release(row)
                self._finish(req, req.finish_reason)
            return True
        return False

    def _decode(self) -> None:
        while self.running and not all(self.backend.can_grow(row) for row in self.running):
            if len(self.running) == 1:
                row, req = next(iter(self.running.items()))
                self._release(row)
                self._fail(req, QueueFull("sequence outgrew the KV memory"))
                return
            self._retract_one()
        if not self.running:
            return
        rows = sorted(self.running)
        try:
            out = self.backend.decode(rows)
        except Exception as exc:
            self.healthy = False
            for row, req in list(self.running.items()):
                self._release(row)
                self._fail(req, BackendFailure(str(exc)))
            for req in list(self.waiting):
                self.waiting.remove(req)
                self._fail(req, BackendFailure(str(exc)))
            return
        self.stats.decode_steps += 1
        self.new_token_ratio = max(MIN_NEW_TOKEN_RATIO, self.new_token_ratio -
                                   (INITIAL_NEW_TOKEN_RATIO - MIN_NEW_TOKEN_RATIO) / RATIO_DECAY_STEPS)
        for row in rows:
            req = self.running.get(row)
            if req is None:
                continue
            produced = out[row] if isinstance(out[row], (list, tuple)) else [out[row]]
            for tok in produced:  # an MTP cycle confirms several tokens; a stop token or the length cap ends early
                self.stats.decode_tokens += 1
                if self._accept_token(req, tok):
                    self._snapshot(req)
                    self._release(row)
                    self._finish(req, req.finish_reason)
                    break

    def step(self) -> bool:
        """One scheduling step (a prefill or a batched decode).  Returns False when there was nothing to do."""
        if not self.healthy:
            return False
        self._expire()
        did = False
        if self.waiting and (not self._decode_next or not self.running):
            did = self._try_prefill()
            self._decode_next = True  # alternate: the next step decodes, if anything is running
        if not did and self.running:
            self._decode()
            self._decode_next = False
            did = True
        return did

    def run_until_idle(self, max_steps: int = 1_000_000) -> None:
        steps = 0
        while not self.idle and self.healthy and steps < max_steps:
            if not self.step():
                break
            steps += 1

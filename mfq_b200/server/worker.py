"""Worker processes: a model served by a child runtime, watched and revived by the front end.

The front end (HTTP server, tokenizer, request queue) stays alive whatever happens to the process that owns the GPU:
a model can run in a child ``mfq runtime --transport stdio`` and the front end talks to it in frames.
:class:`WorkerScheduler` stands where a :class:`~mfq_b200.engine.scheduler.ContinuousBatchScheduler` stands in
:class:`~mfq_b200.server.service.ModelService` (``submit`` / ``cancel`` / ``step`` / ``idle`` / ``healthy``): it sends
each request as a ``generate`` frame with the exact token ids, turns the child's ``token`` frames back into scheduler
events, and enforces queue capacity itself.  Batching, KV memory and retraction are the child's business.

Failure handling (all on the host):

* the child's exit is noticed by ``poll()`` in every ``step`` (and by the reader thread hitting end-of-file): every
  request in flight fails at once with ``backend_failure`` (retryable) instead of waiting for its deadline;
* the next ``submit`` revives the worker -- a fresh child, waited for until its ``ready`` frame -- unless the last
  start is more recent than the back-off (1 s, doubling per consecutive failure up to 60 s), in which case the request
  is refused with ``backend_failure``; a worker that served a request successfully resets the back-off;
* a child that starts but never says ``ready`` within ``ready_timeout`` counts as a failed start and is killed;
* a child that is alive but sends no frame for ``stall_timeout`` seconds while requests are in flight is taken for hung:
  it is killed and handled like a dead one; a request whose own deadline passed without an answer fails with
  ``runtime_deadline_exceeded`` and is cancelled at the child.

Reference: the Python runtime pool launches native workers, polls them until healthy, detects their death with
``process.poll()`` and revives dead or unhealthy runtimes on the next request with a per-model back-off
(``mfq/server/runtime/native.py:245-312``, ``mfq/server/runtime/runtime_pool.py:3394-3426``).
"""

from __future__ import annotations

import itertools
import json
import queue
import subprocess
import threading
import time

from ..engine.scheduler import BackendFailure, Event, QueueFull, Request, SchedulerStats


class WorkerProcess:
    """One child runtime and a thread that reads its frames."""

    def __init__(self, command: list[str], env: dict | None = None, ready_timeout: float = 600.0) -> None:
        self.proc = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1, env=env)
        self.frames: "queue.Queue[dict | None]" = queue.Queue()
        self._lock = threading.Lock()
        threading.Thread(target=self._read, daemon=True).start()
        try:
            first = self.frames.get(timeout=ready_timeout)
        except queue.Empty:
            first = None
        if not first or first.get("type") != "ready":
            self.kill()
            raise BackendFailure(f"worker did not become ready (exit code {self.proc.poll()})")
        self.ready = first

    def _read(self) -> None:
        try:
            for line in self.proc.stdout:
                line = line.strip()
                if line.startswith("{"):
                    try:
                        self.frames.put(json.loads(line))
                    except ValueError:
                        pass
        finally:
            self.frames.put(None)  # end of stream: the child is gone (or closed its output)

    @property
    def alive(self) -> bool:
        return self.proc.poll() is None

    def send(self, frame: dict) -> bool:
        try:
            with self._lock:
                self.proc.stdin.write(json.dumps({"v": 1, **frame}) + "\n")
                self.proc.stdin.flush()
            return True
        except (BrokenPipeError, OSError, ValueError):
            return False

    def kill(self) -> None:
        if self.proc.poll() is None:
            self.proc.kill()
        try:
            self.proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            pass

    def close(self) -> None:
        if self.alive and self.send({"op": "shutdown"}):
            try:
                self.proc.stdin.close()
                self.proc.wait(timeout=30)
                return
            except (subprocess.TimeoutExpired, OSError):
                pass
        self.kill()


class WorkerScheduler:
    def __init__(self, command: list[str], *, capacity: int = 32, max_queue: int = 256, env: dict | None = None,
                 ready_timeout: float = 600.0, backoff: float = 1.0, max_backoff: float = 60.0,
                 clock=time.monotonic, start: bool = True, stall_timeout: float | None = 300.0) -> None:
        self.command, self.env, self.ready_timeout = list(command), env, ready_timeout
        self.capacity, self.max_queue, self.clock = capacity, max_queue, clock
        self.backoff0, self.max_backoff = backoff, max_backoff
        self.stall_timeout = stall_timeout  # requests in flight and no frame for this long: the child hangs -> kill it
        self._last_frame = clock()
        self.stats = SchedulerStats()
        self.running: dict[int, Request] = {}  # request id -> request in flight at the worker
        self.waiting: list[Request] = []       # kept for the status view; the worker queues for itself
        self.healthy = False
        self.worker: WorkerProcess | None = None
        self.failures = 0        # consecutive failed starts / deaths
        self.restarts = 0
        self._last_start = -1e18
        self._ids = itertools.count(1)
        if start:
            self._start()

    # ---- life cycle ------------------------------------------------------------------------------------------------
    def _start(self) -> None:
        self._last_start = self.clock()
        try:
            self.worker = WorkerProcess(self.command, self.env, self.ready_timeout)
        except (BackendFailure, OSError) as exc:
            self.worker, self.healthy = None, False
            self.failures += 1
            raise BackendFailure(f"worker start failed: {exc}") from None
        self.healthy = True

    def _revive_if_due(self) -> None:
        if self.worker is not None and self.worker.alive and self.healthy:
            return
        wait = min(self.max_backoff, self.backoff0 * (2 ** max(0, self.failures - 1))) if self.failures else 0.0
        since = self.clock() - self._last_start
        if since < wait:
            raise BackendFailure(f"worker is down; next start in {wait - since:.1f} s")
        if self.worker is not None:
            self.worker.kill()
        self.restarts += 1
        self._start()

    def _worker_died(self) -> None:
        """Fail everything in flight; the next submit decides about a restart."""
        self.healthy = False
        self.failures += 1
        code = self.worker.proc.poll() if self.worker is not None else None
        for req in list(self.running.values()):
            req.finished, req.finish_reason = True, "backend_failure"
            req.error = BackendFailure(f"worker exited (code {code}) with the request in flight")
            self.stats.failed += 1
            if req.on_event:
                req.on_event(Event("failed", req.id, error_code="backend_failure"))
        self.running.clear()

    def shutdown(self) -> None:
        if self.worker is not None:
            self.worker.close()
        self.healthy = False

    # ---- scheduler interface ---------------------------------------------------------------------------------------
    @property
    def idle(self) -> bool:
        return not self.running

    def submit(self, req: Request) -> int:
        if len(self.running) >= self.capacity + self.max_queue:
            raise QueueFull(f"worker queue is full ({len(self.running)} requests in flight)")
        self._revive_if_due()
        req.id = next(self._ids)
        req.arrival = self.clock()
        p = req.params
        frame = {"id": f"w{req.id}", "op": "generate", "params": {
            "input": {"token_ids": list(req.prompt)}, "stream": False, "stream_tokens": True, "priority": req.priority,
            "timeout_seconds": req.timeout_seconds, "response_format": p.response_format, "logit_bias": p.logit_bias,
            "sampling": {"temperature": p.temperature, "top_p": p.top_p, "top_k": p.top_k, "max_new_tokens": p.max_tokens,
                         "seed": p.seed, "enable_mtp": p.enable_mtp, "presence_penalty": p.presence_penalty,
                         "frequency_penalty": p.frequency_penalty, "repetition_penalty": p.repetition_penalty,
                         "stop_token_ids": list(p.stop_token_ids)}}}
        if not self.running:
            self._last_frame = self.clock()  # the silence before this request does not count against the child
        if req.timeout_seconds:
            req.deadline = req.arrival + float(req.timeout_seconds)
        self.running[req.id] = req
        if not self.worker.send(frame):
            self._worker_died()
            raise BackendFailure("worker went away while the request was being sent")
        self.stats.admitted += 1
        return req.id

    def cancel(self, request_id: int) -> bool:
        if request_id not in self.running or self.worker is None:
            return False
        return self.worker.send({"op": "cancel", "params": {"target": f"w{request_id}"}})

    def step(self) -> bool:
        """Drain the worker's frames into request events; returns True if anything happened."""
        w = self.worker
        if w is None:
            return False
        busy = False
        while True:
            try:
                frame = w.frames.get_nowait()
            except queue.Empty:
                break
            busy = True
            self._last_frame = self.clock()
            if frame is None:  # end of the child's output
                if self.healthy:
                    self._worker_died()
                return True
            rid = str(frame.get("id") or "")
            req = self.running.get(int(rid[1:])) if rid.startswith("w") and rid[1:].isdigit() else None
            if req is None:
                continue
            kind = frame.get("type")
            if kind == "token":
                tok = int(frame["data"]["id"])
                if req.first_token_time is None:
                    req.first_token_time = self.clock()
                req.generated.append(tok)
                self.stats.decode_tokens += 1
                if req.on_event:
                    req.on_event(Event("token", req.id, token=tok))
            elif kind == "result":
                req.finish_reason = frame["data"].get("finish_reason", "stop")
            elif kind == "error":
                req.error = BackendFailure(frame.get("error", {}).get("message", "worker error"))
                req.finish_reason = frame.get("error", {}).get("code", "error")
            elif kind == "done":
                self.running.pop(req.id, None)
                req.finished = True
                if req.error is not None:
                    self.stats.failed += 1
                    if req.on_event:
                        req.on_event(Event("failed", req.id, error_code=req.finish_reason))
                else:
                    self.stats.completed += 1
                    self.failures = 0  # a served request: the worker is fine, forget earlier trouble
                    if req.on_event:
                        req.on_event(Event("completed", req.id, finish_reason=req.finish_reason or "stop"))
        if self.healthy and not w.alive and w.frames.empty():
            self._worker_died()
            busy = True
        now = self.clock()
        for req in [r for r in self.running.values() if r.deadline is not None and now > r.deadline + 1.0]:
            # the child enforces deadlines itself; this is the front end's own bound in case it does not answer
            self.running.pop(req.id, None)
            self.worker.send({"op": "cancel", "params": {"target": f"w{req.id}"}})
            req.finished, req.finish_reason = True, "runtime_deadline_exceeded"
            self.stats.failed += 1
            if req.on_event:
                req.on_event(Event("failed", req.id, error_code="runtime_deadline_exceeded"))
            busy = True
        if self.healthy and self.running and self.stall_timeout and now - self._last_frame > self.stall_timeout:
            w.kill()  # alive but silent with work in flight: a hung engine; the next request starts a fresh child
            self._worker_died()
            busy = True
        return busy

"""Worker processes: requests proxied to a child runtime; its death fails requests at once; the next request revives it."""

import queue
import sys
import time

import pytest

from mfq_b200.cli import main
from mfq_b200.engine.scheduler import BackendFailure, SamplingParams
from mfq_b200.server import ModelService
from mfq_b200.server.tokenizer import ByteTokenizer
from mfq_b200.server.worker import WorkerScheduler


def _collect(events, timeout=120):
    toks, end = [], None
    deadline = time.time() + timeout
    while time.time() < deadline:
        try:
            ev = events.get(True, 0.25)
        except queue.Empty:
            continue
        if ev.kind == "token":
            toks.append(ev.token)
        else:
            end = ev
            break
    return toks, end


def test_requests_run_in_a_child_that_is_revived_after_it_dies(tmp_path):
    ckpt = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--format", "nint8"]) == 0
    command = [sys.executable, "-m", "mfq_b200.cli", "runtime", "--model", str(ckpt), "--device", "cpu",
               "--continuous-batching", "2", "--ctx-size", "512"]
    service = ModelService(max_queue=4, queue_timeout=5.0)
    tok = ByteTokenizer(1024)
    lm = service.add_worker_model("tiny", command, tok, capacity=2, backoff=0.0, ready_timeout=240)
    try:
        prompt = tok.encode("hello worker")
        _req, events = service.submit(lm, prompt, SamplingParams(max_tokens=6))
        toks, end = _collect(events)
        assert end.kind == "completed" and 1 <= len(toks) <= 6
        _req2, events2 = service.submit(lm, prompt, SamplingParams(max_tokens=6))
        assert _collect(events2)[0] == toks  # greedy: the child is deterministic
        # a long request; the child is killed once it has produced a token
        _req3, events3 = service.submit(lm, prompt, SamplingParams(max_tokens=400))
        first = events3.get(True, 120)
        assert first.kind == "token"
        lm.scheduler.worker.proc.kill()
        _more, end = _collect(events3)
        assert end.kind == "failed" and end.error_code == "backend_failure"
        deadline = time.time() + 10
        while lm.scheduler.healthy and time.time() < deadline:
            time.sleep(0.05)
        status = service.status()["instances"][0]
        assert status["healthy"] is False and status["worker_failures"] == 1
        # the next request starts a fresh child and is served
        _req4, events4 = service.submit(lm, prompt, SamplingParams(max_tokens=6))
        toks4, end4 = _collect(events4)
        assert end4.kind == "completed" and toks4 == toks
        status = service.status()["instances"][0]
        assert status["healthy"] is True and status["worker_restarts"] == 1 and status["worker_failures"] == 0
    finally:
        service.shutdown()
    assert lm.scheduler.worker.proc.poll() is not None  # the child went down with the service


def test_failed_starts_back_off():
    now = [100.0]
    sched = WorkerScheduler([sys.executable, "-c", "pass"], ready_timeout=30, backoff=4.0, clock=lambda: now[0], start=False)
    from mfq_b200.engine.scheduler import Request
    with pytest.raises(BackendFailure, match="start failed"):
        sched.submit(Request([1, 2, 3]))
    assert sched.failures == 1 and not sched.healthy
    now[0] += 1.0
    with pytest.raises(BackendFailure, match="next start in 3.0 s"):
        sched.submit(Request([1, 2, 3]))
    assert sched.failures == 1  # refused without another start
    now[0] += 3.5
    with pytest.raises(BackendFailure, match="start failed"):
        sched.submit(Request([1, 2, 3]))
    assert sched.failures == 2 and sched.restarts == 2
    now[0] += 5.0  # the back-off doubled to 8 s
    with pytest.raises(BackendFailure, match="next start in 3.0 s"):
        sched.submit(Request([1, 2, 3]))


_SILENT_CHILD = (
    "import sys, json, time\n"
    "print(json.dumps({'v': 1, 'type': 'ready', 'data': {'models': ['m']}}), flush=True)\n"
    "for line in sys.stdin:\n"
    "    pass\n"  # reads requests, never answers
)


def test_a_silent_child_is_killed_and_deadlines_are_enforced_by_the_front_end():
    from mfq_b200.engine.scheduler import Request
    events = []
    sched = WorkerScheduler([sys.executable, "-c", _SILENT_CHILD], ready_timeout=60, stall_timeout=3.0, backoff=0.0)
    try:
        late = Request([1, 2, 3], timeout_seconds=0.2, on_event=events.append)
        stuck = Request([4, 5, 6], on_event=events.append)
        sched.submit(late)
        sched.submit(stuck)
        deadline = time.time() + 20
        while sched.running and time.time() < deadline:
            sched.step()
            time.sleep(0.05)
        kinds = [(e.request_id, e.kind, e.error_code) for e in events]
        assert (late.id, "failed", "runtime_deadline_exceeded") in kinds
        assert (stuck.id, "failed", "backend_failure") in kinds
        assert not sched.healthy and sched.failures == 1 and sched.worker.proc.poll() is not None  # the hung child was killed
    finally:
        sched.shutdown()

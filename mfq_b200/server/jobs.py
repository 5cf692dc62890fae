"""Background jobs of the control API: quantize / evaluate / benchmark / calibrate / inspect / diagnose runs as child processes of the server.

A job is one ``mfq`` command line.  Its combined output goes to a log file whose tail the API returns; a job is stopped
by signalling exactly the process the manager started (never by name).  Finished jobs stay listed until they are
deleted.  Reference: ``mfq/server/services/jobs.py`` and ``tool_jobs.py`` (quantize / eval / benchmark jobs).
"""

from __future__ import annotations

import subprocess
import sys
import tempfile
import threading
import time
import uuid
from dataclasses import dataclass, field
from pathlib import Path

ALLOWED = ("quantize", "eval", "inspect", "diagnose", "calibrate", "solve-ew", "bench", "optimize-layout", "wt2-reference")


@dataclass
class Job:
    id: str
    kind: str
    argv: list[str]
    log_path: Path
    proc: subprocess.Popen | None = None
    created: float = field(default_factory=time.time)
    finished: float | None = None
    cancelled: bool = False

    @property
    def state(self) -> str:
        if self.proc is None:
            return "failed"
        rc = self.proc.poll()
        if rc is None:
            return "running"
        if self.finished is None:
            self.finished = time.time()
        return "cancelled" if self.cancelled else ("succeeded" if rc == 0 else "failed")

    def describe(self, tail_bytes: int = 4096) -> dict:
        state = self.state
        data = ""
        if tail_bytes > 0:  # 0 = no log text at all (the listing route); never read more than the tail
            try:
                with open(self.log_path, "rb") as f:
                    f.seek(0, 2)
                    f.seek(max(0, f.tell() - tail_bytes))
                    data = f.read(tail_bytes).decode("utf-8", errors="replace")
            except OSError:
                data = ""
        return {"id": self.id, "kind": self.kind, "argv": self.argv, "state": state, "created": self.created,
                "finished": self.finished, "exit_code": self.proc.poll() if self.proc else None, "log_tail": data}


class JobManager:
    def __init__(self, log_dir=None, max_running: int = 2, launcher: list[str] | None = None) -> None:
        self.log_dir = Path(log_dir) if log_dir else Path(tempfile.mkdtemp(prefix="mfq-jobs-"))
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self.max_running = max_running
        self.launcher = launcher or [sys.executable, "-m", "mfq_b200.cli"]
        self.jobs: dict[str, Job] = {}
        self._lock = threading.Lock()

    def submit(self, kind: str, args: list[str]) -> Job:
        if kind not in ALLOWED:
            raise ValueError(f"unknown job kind {kind!r} (one of {', '.join(ALLOWED)})")
        if not all(isinstance(a, str) for a in args):
            raise ValueError("job arguments must be strings")
        with self._lock:
            if sum(j.state == "running" for j in self.jobs.values()) >= self.max_running:
                raise RuntimeError("too many running jobs")
            jid = uuid.uuid4().hex[:12]
            job = Job(jid, kind, [kind, *args], self.log_dir / f"{jid}.log")
            with open(job.log_path, "wb") as log:
                job.proc = subprocess.Popen(self.launcher + job.argv, stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL)
            self.jobs[jid] = job
            return job

    def cancel(self, jid: str) -> bool:
        job = self.jobs.get(jid)
        if job is None or job.proc is None or job.proc.poll() is not None:
            return False
        job.cancelled = True
        job.proc.terminate()  # exactly the child this manager started
        try:
            job.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            job.proc.kill()
        return True

    def delete(self, jid: str) -> bool:
        job = self.jobs.get(jid)
        if job is None or job.state == "running":
            return False
        del self.jobs[jid]
        job.log_path.unlink(missing_ok=True)
        return True

    def shutdown(self) -> None:
        for jid in list(self.jobs):
            self.cancel(jid)

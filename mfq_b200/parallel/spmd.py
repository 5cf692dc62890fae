"""Serving a tensor-parallel model: one scheduler, every rank's engine in lockstep.

Tensor (and expert) parallel engines are SPMD: every rank must make the same engine calls in the same order, because
each call launches kernels whose collectives meet the other ranks' kernels.  The request scheduler, the tokenizer and
the HTTP server live on rank 0 only.  So rank 0 wraps its engine in a :class:`LeaderBackend`: every state-changing call
of the scheduler's back-end protocol (``prefill``, ``decode``, ``can_grow``, ``release``, ``set_sampling``,
``save_session``) is first appended to a command log in the job's key-value store, then executed locally; the other
ranks sit in :func:`follower_loop`, read the log in order and make the same call on their own engine.  Page allocation,
sampling (seeded) and row bookkeeping are deterministic, so all ranks stay bit-identical without exchanging state.

* The log is a ``torch.distributed`` store (the rendezvous TCP store of the job, or a ``HashStore`` for in-process
  tests), not a collective: an idle server never trips a collective timeout, and a follower waits in short slices so it
  notices a shutdown or a dead leader (heartbeat key) instead of blocking forever.
* A follower that fails a call records the error under ``spmd/error/<rank>`` and leaves its loop.  The leader checks
  for such records before every command and raises :class:`~mfq_b200.engine.scheduler.BackendFailure`, which latches
  the scheduler unhealthy (requests fail fast instead of waiting for a collective that can no longer complete).  The
  collectives themselves have bounded device-side waits that report through the status word.

The reference runs its tensor-parallel ranks as threads of one process around a primary GPU
(``cpp_runtime/backends/cuda/parallel``); with one process per GPU this command log takes the place of its in-process
task fan-out.
"""

from __future__ import annotations

import pickle
import time

from ..engine.scheduler import BackendFailure

REPLICATED = ("prefill", "decode", "can_grow", "release", "set_sampling", "save_session", "grow")
_PREFIX = "spmd"


class CommandLog:
    """Append-only, single-writer log of pickled commands in a distributed store."""

    def __init__(self, store, rank: int, world: int) -> None:
        self.store, self.rank, self.world = store, rank, world
        self.next = 0  # index of the next command to write (leader) / read (follower)

    # ---- leader ------------------------------------------------------------------------------------------------------
    def append(self, command: tuple) -> None:
        self.store.set(f"{_PREFIX}/cmd/{self.next}", pickle.dumps(command))
        self.next += 1
        if self.next % 256 == 0:
            self._trim()

    def _trim(self) -> None:
        """Delete commands that every follower has acknowledged."""
        done = min((int(self.store.add(f"{_PREFIX}/ack/{r}", 0)) for r in range(1, self.world)), default=self.next)
        start = int(self.store.add(f"{_PREFIX}/trimmed", 0))
        for i in range(start, done):
            self.store.delete_key(f"{_PREFIX}/cmd/{i}")
        if done > start:
            self.store.add(f"{_PREFIX}/trimmed", done - start)

    def follower_errors(self) -> dict[int, str]:
        out = {}
        for r in range(1, self.world):
            key = f"{_PREFIX}/error/{r}"
            if self.store.check([key]):
                out[r] = self.store.get(key).decode(errors="replace")
        return out

    def beat(self) -> None:
        self.store.set(f"{_PREFIX}/leader_beat", str(time.time()))

    # ---- follower ----------------------------------------------------------------------------------------------------
    def read(self, poll_seconds: float = 1.0, leader_timeout: float | None = None):
        """Next command, or None when the leader's heartbeat is older than ``leader_timeout`` seconds."""
        from datetime import timedelta
        key = f"{_PREFIX}/cmd/{self.next}"
        while True:
            try:
                self.store.wait([key], timedelta(seconds=poll_seconds))
                break
            except Exception:  # the store's wait timed out (its exception type differs between store kinds)
                if leader_timeout is not None and self.store.check([f"{_PREFIX}/leader_beat"]):
                    if time.time() - float(self.store.get(f"{_PREFIX}/leader_beat")) > leader_timeout:
                        return None
        command = pickle.loads(self.store.get(key))
        self.next += 1
        self.store.add(f"{_PREFIX}/ack/{self.rank}", 1)
        return command

    def fail(self, message: str) -> None:
        self.store.set(f"{_PREFIX}/error/{self.rank}", message)


class LeaderBackend:
    """Rank 0's engine as the scheduler sees it: replicated calls go to the log first."""

    def __init__(self, engine, log: CommandLog) -> None:
        self._engine, self._log = engine, log
        log.beat()

    def __getattr__(self, name):
        target = getattr(self._engine, name)
        if name not in REPLICATED:
            return target

        def call(*args, **kwargs):
            errors = self._log.follower_errors()
            if errors:
                raise BackendFailure(f"rank(s) {sorted(errors)} failed: {next(iter(errors.values()))}")
            self._log.append((name, _plain(args), _plain(kwargs)))
            self._log.beat()
            return target(*args, **kwargs)
        return call

    def shutdown_followers(self) -> None:
        self._log.append(("__shutdown__", (), {}))


def _plain(value):
    """Tensors travel as lists (prompts are short id lists; nothing large goes through the log)."""
    import torch
    if isinstance(value, torch.Tensor):
        return value.tolist()
    if isinstance(value, tuple):
        return tuple(_plain(v) for v in value)
    if isinstance(value, list):
        return [_plain(v) for v in value]
    if isinstance(value, dict):
        return {k: _plain(v) for k, v in value.items()}
    return value


def follower_loop(engine, log: CommandLog, poll_seconds: float = 1.0, leader_timeout: float | None = 120.0) -> str:
    """Mirror the leader's engine calls until it shuts down.  Returns why the loop ended:
    ``"shutdown"``, ``"leader_lost"`` or ``"error"``."""
    while True:
        command = log.read(poll_seconds, leader_timeout)
        if command is None:
            return "leader_lost"
        name, args, kwargs = command
        if name == "__shutdown__":
            return "shutdown"
        try:
            getattr(engine, name)(*args, **kwargs)
        except Exception as exc:  # this rank can no longer follow: tell the leader and stop
            log.fail(f"{type(exc).__name__}: {exc}")
            return "error"

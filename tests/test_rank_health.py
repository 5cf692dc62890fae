"""Rank failure detection and group re-forming, with the failure injected on the host (gloo ranks on the CPU)."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from mfq_b200.parallel.health import RankFailure, RankHealth


class FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_heartbeat_timeout_and_failure_report():
    now = [100.0]
    store = FakeStore()
    h = [RankHealth(store, r, 3, timeout=5.0, clock=lambda: now[0]) for r in range(3)]
    h[0].check()
    now[0] = 104.0
    h[1].beat()
    h[2].beat()
    now[0] = 108.0  # everyone beat within 5 s of now except nobody: rank 0's own beat is not checked by itself
    h[0].check()
    now[0] = 110.5
    with pytest.raises(RankFailure) as e:
        h[0].check()
    assert sorted(e.value.failed) == [1, 2] and "no heartbeat" in e.value.failed[1]
    h[1].beat()
    h[2].report_failure("status word 4: a peer wait timed out")
    with pytest.raises(RankFailure) as e:
        h[0].check()
    assert list(e.value.failed) == [2] and "status word" in e.value.failed[2] and h[0].survivors() == [0, 1]
    late = RankHealth(FakeStore(), 0, 2, timeout=5.0, clock=lambda: now[0])
    assert late.failed() == {1: "never joined"}


def test_ranks_survive_a_peer_that_leaves_between_steps():
    env = dict(os.environ, VICTIM="2", FAIL_STEP="3", STORE_PORT="29731")
    procs = []
    for rank in range(3):
        e = dict(env, RANK=str(rank), WORLD_SIZE="3")
        procs.append(subprocess.Popen([sys.executable, str(Path(__file__).with_name("health_worker.py"))], env=e,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=120) for p in procs]
    results = {}
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-2000:]
        line = [l for l in out.splitlines() if l.startswith("HEALTH_RESULT ")][-1]
        r = json.loads(line[len("HEALTH_RESULT "):])
        results[r["rank"]] = r
    assert results[2] == {"rank": 2, "left_at": 3}
    for r in (0, 1):
        assert results[r]["detected"] == [2] and results[r]["world_after"] == 2
        # three steps with ranks 1+2+3, then three steps of the re-formed group with ranks 1+2
        assert results[r]["sums"] == [6.0, 6.0, 6.0, 3.0, 3.0, 3.0]

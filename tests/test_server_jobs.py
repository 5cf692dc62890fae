"""Jobs API: an mfq command runs as a child process of the server; status, log tail, cancel, delete."""

import sys
import time

from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.jobs import JobManager


def _wait(fn, timeout=60.0):
    end = time.time() + timeout
    while time.time() < end:
        v = fn()
        if v:
            return v
        time.sleep(0.1)
    raise AssertionError("timed out")


def test_job_lifecycle_over_http():
    service = ModelService()
    with TestClient(create_app(service)) as c:
        assert c.post("/api/v1/jobs", json={"kind": "rm", "args": []}).status_code == 400
        r = c.post("/api/v1/jobs", json={"kind": "diagnose", "args": ["--check", "container"]})
        assert r.status_code == 202
        jid = r.json()["id"]
        done = _wait(lambda: (lambda j: j if j["state"] != "running" else None)(c.get(f"/api/v1/jobs/{jid}").json()))
        assert done["state"] == "succeeded" and '"container"' in done["log_tail"] and done["exit_code"] == 0
        assert [j["id"] for j in c.get("/api/v1/jobs").json()["jobs"]] == [jid]
        assert c.delete(f"/api/v1/jobs/{jid}").json() == {"deleted": True}
        assert c.get(f"/api/v1/jobs/{jid}").status_code == 404
    service.shutdown()


def test_cancel_stops_exactly_the_child(tmp_path):
    # a launcher that sleeps stands in for a long quantization
    jm = JobManager(tmp_path, max_running=1, launcher=[sys.executable, "-c", "import time,sys; print('started', flush=True); time.sleep(60)"])
    job = jm.submit("quantize", ["in", "out"])
    _wait(lambda: "started" in job.describe()["log_tail"])
    try:
        jm.submit("inspect", ["x"])
        raise AssertionError("the running-job cap was not enforced")
    except RuntimeError:
        pass
    pid = job.proc.pid
    assert jm.cancel(job.id) and job.state == "cancelled" and job.proc.pid == pid
    assert not jm.cancel(job.id)
    assert jm.delete(job.id) and not jm.jobs

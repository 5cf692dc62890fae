"""`mfq serve` as a process on a tiny CPU checkpoint: health, a JSON-constrained completion, policies on disk, clean exit."""

import json
import os
import signal
import subprocess
import sys
import time
import urllib.request

from mfq_b200.cli import main
from mfq_b200.server.tp_serve import free_port


def _call(url, body=None, method=None, timeout=120):
    data = json.dumps(body).encode() if body is not None else None
    req = urllib.request.Request(url, data=data, method=method, headers={"content-type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def test_single_process_server(tmp_path):
    ckpt = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--format", "nint8"]) == 0
    port, data = free_port(), tmp_path / "data"
    log = open(tmp_path / "serve.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "mfq_b200.cli", "serve", "--model", str(ckpt), "--backend", "cpu", "--port", str(port),
                             "--max-requests-per-runtime", "2", "--context-size", "256", "--data-dir", str(data),
                             "--prefill-chunk-size", "64", "--log-level", "warning"], stdout=log, stderr=subprocess.STDOUT)
    try:
        base = f"http://127.0.0.1:{port}"
        deadline = time.time() + 240
        while True:
            try:
                assert _call(base + "/health", timeout=2)["status"] == "ok"
                break
            except Exception:
                assert proc.poll() is None and time.time() < deadline, (tmp_path / "serve.log").read_text()[-3000:]
                time.sleep(1.0)
        out = _call(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": "json please"}], "max_tokens": 40,
                                                     "response_format": {"type": "json_object"}, "session_id": "s"})
        text = out["choices"][0]["message"]["content"]
        assert text.lstrip().startswith("{")
        if out["choices"][0]["finish_reason"] == "stop":
            assert isinstance(json.loads(text), dict)
        assert _call(base + "/api/v1/runtime/policies/tiny", {"inference": {"max_tokens": 3}}, method="PUT")["policy"]["inference"]["max_tokens"] == 3
        short = _call(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}]})
        assert short["usage"]["completion_tokens"] <= 3
        assert json.loads((data / "policies.json").read_text())["tiny"]["inference"]["max_tokens"] == 3
        assert (data / "mfq-server.sqlite3").exists()
        metrics = urllib.request.urlopen(base + "/metrics", timeout=10).read().decode()
        assert "mfq_runtime_kv_bytes{" in metrics and "mfq_requests_total{" in metrics
    finally:
        proc.send_signal(signal.SIGINT)
        try:
            assert proc.wait(timeout=60) == 0
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.wait(timeout=30)
            raise
        finally:
            log.close()

"""`mfq serve --tensor-parallel 2` end to end on CPU ranks (gloo): launcher, sharded load, command log, HTTP on rank 0."""

import json
import os
import signal
import subprocess
import sys
import time
import urllib.request

from mfq_b200.cli import main
from mfq_b200.server.tp_serve import free_port, launcher_argv


def _post(url, body, timeout=120):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"content-type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def test_launcher_command_line():
    argv = launcher_argv(["serve", "--model", "m.mfq", "--tensor-parallel", "4"], 4, port=29555)
    assert argv[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"] and "--nproc-per-node=4" in argv
    assert argv[argv.index("--master-addr") + 1] == "127.0.0.1" and argv[argv.index("--master-port") + 1] == "29555"
    assert argv[-7:] == ["-m", "mfq_b200.cli", "serve", "--model", "m.mfq", "--tensor-parallel", "4"]


import pytest


@pytest.mark.parametrize("mode", [["--tensor-parallel", "2"], ["--layer-parallel", "2"]])
def test_two_cpu_ranks_serve_a_completion(tmp_path, mode):
    serve_and_complete(tmp_path, mode, ["--device", "cpu"], {"OMP_NUM_THREADS": "2"})


def serve_and_complete(tmp_path, mode, device_args, env_extra):
    """Start `mfq serve` with ``mode`` on a tiny checkpoint, wait for /health, run the same greedy completion twice (the second
    one resumes the session), check the runtime status, stop the server."""
    ckpt = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--full-precision"]) == 0
    port = free_port()
    env = dict(os.environ, **env_extra)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    log = open(tmp_path / "serve.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "mfq_b200.cli", "serve", "--model", str(ckpt), *device_args, "--port", str(port),
                             *mode, "--continuous-batching", "2", "--ctx-size", "96"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    try:
        base = f"http://127.0.0.1:{port}"
        deadline = time.time() + 240
        while True:
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    assert json.loads(r.read())["status"] == "ok"
                break
            except Exception:
                assert proc.poll() is None, (tmp_path / "serve.log").read_text()[-3000:]
                assert time.time() < deadline, (tmp_path / "serve.log").read_text()[-3000:]
                time.sleep(1.0)
        body = {"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0, "session_id": "s1"}
        a = _post(base + "/v1/chat/completions", body)
        b = _post(base + "/v1/chat/completions", body)
        assert a["usage"]["completion_tokens"] >= 1 and a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
        status = json.loads(urllib.request.urlopen(base + "/api/v1/runtime/status", timeout=10).read())
        assert status["instances"][0]["healthy"] is True
    finally:
        os.killpg(proc.pid, signal.SIGINT)
        try:
            proc.wait(timeout=60)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
            proc.wait(timeout=30)
        log.close()

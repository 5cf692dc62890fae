"""stdio NDJSON transport over the model service (fake back end)."""

import io
import json

from mfq_b200.server import ModelService
from mfq_b200.server.stdio import StdioTransport
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend as _Echo


class EchoBackend(_Echo):
    """Keeps one script per row, so that concurrent requests do not reset each other."""

    def prefill(self, row, tokens, params):
        scripts = dict(getattr(self, "script", {}))
        first = super().prefill(row, tokens, params)
        scripts[row] = self.script[row]
        self.script = scripts
        return first


def _run(frames):
    service = ModelService(max_queue=4, queue_timeout=5.0)
    backend = EchoBackend(max_batch=2)
    service.add_model("echo", backend, ByteTokenizer())
    out = io.StringIO()
    StdioTransport(service, io.StringIO("".join(json.dumps(f) + "\n" for f in frames)), out).serve()
    service.shutdown()
    return [json.loads(l) for l in out.getvalue().splitlines()], backend


def test_generate_stream_status_and_errors():
    frames, backend = _run([
        {"v": 1, "id": "a", "op": "generate", "params": {"model": "echo", "input": {"messages": [{"role": "user", "content": "hi"}]},
                                                       "sampling": {"temperature": 0.0, "max_new_tokens": 8}, "stream": True}},
        {"v": 1, "id": "b", "op": "generate", "params": {"model": "echo", "input": {"benchmark_prompt_tokens": 37},
                                                       "sampling": {"max_new_tokens": 8}, "stream": False}},
        {"v": 1, "id": "c", "op": "generate", "params": {"model": "nope", "input": {"messages": []}}},
        {"v": 1, "id": "s", "op": "status"},
        {"v": 1, "id": "x", "op": "frobnicate"},
        {"v": 1, "op": "shutdown"},
    ])
    assert frames[0]["type"] == "ready" and frames[0]["data"]["models"] == ["echo"] and all(f["v"] == 1 for f in frames)
    by = {}
    for f in frames[1:]:
        by.setdefault(f.get("id"), []).append(f)
    a = by["a"]
    assert "".join(f["data"]["text"] for f in a if f["type"] == "delta") == "ok!"
    res = [f for f in a if f["type"] == "result"][0]["data"]
    assert res["text"] == "ok!" and res["finish_reason"] == "stop" and res["usage"]["completion_tokens"] == 3
    assert {"prefill_ms", "decode_ms", "total_ms"} <= set(res["metrics"]) and a[-1]["type"] == "done"
    b = [f for f in by["b"] if f["type"] == "result"][0]["data"]
    assert b["usage"]["prompt_tokens"] == 37 and not [f for f in by["b"] if f["type"] == "delta"]
    assert by["c"][0]["type"] == "error" and by["c"][0]["error"]["code"] == "model_not_found" and by["c"][-1]["type"] == "done"
    assert by["s"][0]["type"] == "result" and "instances" in by["s"][0]["data"]
    assert by["x"][0]["error"]["code"] == "unknown_op"


def test_runtime_command_over_pipes(tmp_path):
    """`mfq runtime --transport stdio` on a tiny CPU checkpoint: ready frame, one generate, shutdown."""
    import subprocess
    import sys

    from mfq_b200.cli import main
    ckpt = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--format", "nint8"]) == 0
    frames = [{"v": 1, "id": "g", "op": "generate", "params": {"input": {"benchmark_prompt_tokens": 12},
                                                              "sampling": {"max_new_tokens": 4, "temperature": 0.0}}},
              {"v": 1, "op": "shutdown"}]
    proc = subprocess.run([sys.executable, "-m", "mfq_b200.cli", "runtime", "--model", str(ckpt), "--device", "cpu",
                           "--continuous-batching", "2", "--ctx-size", "64"],
                          input="".join(json.dumps(f) + "\n" for f in frames), capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = [json.loads(l) for l in proc.stdout.splitlines()]
    assert out[0]["type"] == "ready" and out[0]["data"]["models"] == ["tiny"]
    res = [f for f in out if f.get("id") == "g" and f["type"] == "result"][0]["data"]
    assert res["usage"]["prompt_tokens"] == 12 and 1 <= res["usage"]["completion_tokens"] <= 4
    assert out[-1] == {"v": 1, "id": "g", "type": "done"}

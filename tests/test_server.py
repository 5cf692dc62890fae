"""HTTP surface with a fake backend: OpenAI / Anthropic shapes, SSE, error envelope and status codes, metrics, auth."""

import json

import pytest
from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.tokenizer import ByteTokenizer
from test_scheduler import FakeBackend


class EchoBackend(FakeBackend):
    """Generates 'ok!' then the stop token."""

    def prefill(self, row, tokens, params):
        super().prefill(row, tokens, params)
        self.script = {row: [ord("o") + 3, ord("k") + 3, ord("!") + 3, 2]}
        return self.script[row].pop(0)

    def decode(self, rows):
        return {r: (self.script[r].pop(0) if self.script[r] else 2) for r in rows}


@pytest.fixture()
def client():
    service = ModelService(max_queue=2, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    with TestClient(create_app(service)) as c:
        yield c, service
    service.shutdown()


def test_health_models_and_chat_completion(client):
    c, _ = client
    assert c.get("/health").json()["model"] == "echo"
    assert c.get("/v1/models").json()["data"][0]["id"] == "echo"
    assert c.get("/v1/models/nope").status_code == 404
    r = c.post("/v1/chat/completions", json={"model": "echo", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 16})
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "chat.completion" and body["choices"][0]["message"]["content"] == "ok!"
    assert body["choices"][0]["finish_reason"] == "stop" and body["usage"]["completion_tokens"] == 3


def test_streaming_chunks(client):
    c, _ = client
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "stream": True,
                                                         "stream_options": {"include_usage": True}}) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert all(ch["object"] == "chat.completion.chunk" for ch in chunks)
    assert "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks) == "ok!"
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["usage"]["completion_tokens"] == 3


def test_stop_string_and_length(client):
    c, _ = client
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "stop": ["k"]}).json()
    assert r["choices"][0]["message"]["content"] == "o" and r["choices"][0]["finish_reason"] == "stop"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 2}).json()
    assert r["choices"][0]["message"]["content"] == "ok" and r["choices"][0]["finish_reason"] == "length"


def test_anthropic_messages(client):
    c, _ = client
    r = c.post("/v1/messages", json={"model": "echo", "max_tokens": 16, "system": "be brief",
                                      "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}]}).json()
    assert r["type"] == "message" and r["content"][0]["text"] == "ok!" and r["stop_reason"] == "end_turn"
    with c.stream("POST", "/v1/messages", json={"max_tokens": 16, "stream": True, "messages": [{"role": "user", "content": "hi"}]}) as s:
        events = [l[7:] for l in s.iter_lines() if l.startswith("event: ")]
    assert events[0] == "message_start" and events[-1] == "message_stop" and "content_block_delta" in events
    assert c.post("/v1/messages/count_tokens", json={}).status_code == 501


def test_error_envelope_and_status_codes(client):
    c, service = client
    assert c.post("/v1/chat/completions", json={"model": "missing", "messages": [{"role": "user", "content": "x"}]}).status_code == 404
    e = c.post("/v1/chat/completions", json={"messages": []}).json()["error"]
    assert set(e) == {"code", "message", "retryable", "details"}
    lm = service.models["echo"]
    lm.scheduler.max_queue = 0
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 429 and r.json()["error"]["code"] == "runtime_queue_full" and r.json()["error"]["retryable"]
    lm.scheduler.max_queue = 4


def test_metrics_and_control_api(client):
    c, _ = client
    c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]})
    text = c.get("/metrics").text
    assert c.get("/metrics").headers["content-type"].startswith("text/plain; version=0.0.4")
    for name in ("mfq_runtime_batch_capacity", "mfq_requests_total", "mfq_request_completion_tokens_total", "mfq_request_ttft_seconds_bucket"):
        assert name in text
    assert 'result="ok"' in text and 'model="echo"' in text
    st = c.get("/api/v1/runtime/status").json()
    assert st["instances"][0]["model"] == "echo" and st["instances"][0]["healthy"]
    assert c.post("/api/v1/models/unload", json={"model": "echo"}).json() == {"unloaded": True}
    assert c.get("/v1/models").json()["data"] == []


def test_api_key():
    service = ModelService()
    service.add_model("echo", EchoBackend(), ByteTokenizer())
    with TestClient(create_app(service, api_key="s3cret")) as c:
        assert c.get("/health").status_code == 200
        assert c.get("/v1/models").status_code == 401
        assert c.get("/v1/models", headers={"authorization": "Bearer s3cret"}).status_code == 200
        assert c.get("/metrics", headers={"x-api-key": "s3cret"}).status_code == 200
    service.shutdown()


def test_sessions_and_sampling_profile(client):
    client, _service = client
    s = client.post("/api/v1/sessions", json={"title": "t1", "model": "tiny"}).json()
    sid = s["id"]
    assert client.post(f"/api/v1/sessions/{sid}/messages", json={"role": "user", "content": "hi"}).json() == {"seq": 0}
    assert client.post(f"/api/v1/sessions/{sid}/messages", json={"role": "assistant", "content": "yo"}).json() == {"seq": 1}
    got = client.get(f"/api/v1/sessions/{sid}").json()
    assert [m["content"] for m in got["messages"]] == ["hi", "yo"] and got["title"] == "t1"
    assert client.patch(f"/api/v1/sessions/{sid}", json={"title": "t2"}).json() == {"renamed": True}
    assert client.get("/api/v1/sessions").json()["sessions"][0]["title"] == "t2"
    assert client.get("/api/v1/sessions/nope").status_code == 404
    assert client.post("/api/v1/sessions/nope/messages", json={"content": "x"}).status_code == 404
    assert client.delete(f"/api/v1/sessions/{sid}").json() == {"deleted": True}
    prof = client.get("/api/v1/runtime/sampling-profile").json()
    assert prof["source"] == "builtin" and prof["chat"]["top_p"] == 1.0

"""Per-model policies: validated, persisted, applied to request defaults and scheduler limits."""

import pytest
from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.policies import PolicyStore, validate
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend


def test_validation_and_persistence(tmp_path):
    assert validate({"inference": {"temperature": 1, "enable_mtp": True}}) == {"inference": {"temperature": 1.0, "enable_mtp": True}}
    for bad in ({"speed": {}}, {"inference": {"temperature": "hot"}}, {"inference": {"enable_mtp": 1}}, {"memory": {"kv_budget_gb": -1}},
                {"context": {"window": 5}}, {"inference": 3}):
        with pytest.raises(ValueError):
            validate(bad)
    path = tmp_path / "state" / "policies.json"
    store = PolicyStore(path)
    store.put("m", {"inference": {"max_tokens": 2, "temperature": 0.5}, "context": {"max_context_tokens": 4096}})
    again = PolicyStore(path)
    assert again.get("m")["context"] == {"max_context_tokens": 4096} and again.get("other") == {}
    body = again.request_defaults("m", {"temperature": 0.0, "messages": []})
    assert body["temperature"] == 0.0 and body["max_tokens"] == 2  # the request's own value wins, gaps are filled
    assert again.request_defaults("m", {"max_completion_tokens": 9}).get("max_tokens") is None
    again.put("m", {})
    assert PolicyStore(path).all() == {}


def test_routes_apply_defaults_and_limits(tmp_path):
    service = ModelService(max_queue=8, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    store = PolicyStore(tmp_path / "p.json")
    with TestClient(create_app(service, policies=store)) as c:
        chat = {"model": "echo", "messages": [{"role": "user", "content": "hi"}]}
        assert c.post("/v1/chat/completions", json=chat).json()["usage"]["completion_tokens"] == 3
        r = c.put("/api/v1/runtime/policies/echo", json={"inference": {"max_tokens": 2}, "concurrency": {"max_queue": 3, "queue_timeout": 1.5}})
        assert r.status_code == 200 and r.json()["policy"]["concurrency"]["max_queue"] == 3
        assert service.models["echo"].scheduler.max_queue == 3 and service.models["echo"].scheduler.queue_timeout == 1.5
        out = c.post("/v1/chat/completions", json=chat).json()
        assert out["usage"]["completion_tokens"] == 2 and out["choices"][0]["finish_reason"] == "length"
        assert c.post("/v1/chat/completions", json=dict(chat, max_tokens=16)).json()["usage"]["completion_tokens"] == 3
        listing = c.get("/api/v1/runtime/policies").json()
        assert listing["policies"]["echo"]["inference"] == {"max_tokens": 2} and "memory" in listing["sections"]
        assert c.get("/api/v1/runtime/policies/echo").json()["policy"]["inference"]["max_tokens"] == 2
        assert c.put("/api/v1/runtime/policies/echo", json={"inference": {"warp": 9}}).status_code == 400
    service.shutdown()

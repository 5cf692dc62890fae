"""API keys with scopes: open without keys, 401 / 403, key management routes, digests on disk."""

import json

from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.auth import KeyStore, required_scope
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend


def test_scope_table():
    assert required_scope("GET", "/health") is None
    assert required_scope("POST", "/v1/chat/completions") == "inference" and required_scope("GET", "/v1/models") == "read"
    assert required_scope("GET", "/api/v1/runtime/status") == "read" and required_scope("POST", "/api/v1/models/load") == "admin"
    assert required_scope("GET", "/api/v1/auth/keys") == "admin" and required_scope("GET", "/metrics") == "read"


def test_keys_and_scopes_over_http(tmp_path):
    store = KeyStore(tmp_path / "keys.json")
    store.add("root-secret", ("admin",), "root")
    service = ModelService(max_queue=2, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    chat = {"model": "echo", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8}
    with TestClient(create_app(service, api_key=store)) as c:
        assert c.get("/health").status_code == 200
        assert c.post("/v1/chat/completions", json=chat).status_code == 401
        admin = {"authorization": "Bearer root-secret"}
        r = c.post("/api/v1/auth/keys", json={"scopes": ["inference"], "name": "app"}, headers=admin)
        key, kid = r.json()["key"], r.json()["id"]
        user = {"x-api-key": key}
        assert c.post("/v1/chat/completions", json=chat, headers=user).status_code == 200
        assert c.get("/api/v1/runtime/status", headers=user).status_code == 403       # no read scope
        assert c.post("/api/v1/models/unload", json={"model": "x"}, headers=user).status_code == 403
        assert c.get("/api/v1/runtime/status", headers=admin).status_code == 200
        listed = c.get("/api/v1/auth/keys", headers=admin).json()["keys"]
        assert [k["name"] for k in listed] == ["root", "app"] and all("key" not in k for k in listed)
        assert c.post("/api/v1/auth/keys", json={"scopes": ["everything"]}, headers=admin).status_code == 400
        assert c.delete(f"/api/v1/auth/keys/{kid}", headers=admin).json() == {"revoked": True}
        assert c.post("/v1/chat/completions", json=chat, headers=user).status_code == 401
    service.shutdown()
    on_disk = json.loads((tmp_path / "keys.json").read_text())
    assert "root-secret" not in json.dumps(on_disk) and len(on_disk) == 1  # digests only
    assert KeyStore(tmp_path / "keys.json").allows("root-secret", "admin")


def test_empty_key_table_does_not_reopen_the_server(tmp_path):
    """A server started with a key or a key file keeps refusing requests when its table is empty."""
    service = ModelService(max_queue=2, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    chat = {"model": "echo", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8}
    with TestClient(create_app(service, api_key="only-key")) as c:
        admin = {"authorization": "Bearer only-key"}
        kid = c.get("/api/v1/auth/keys", headers=admin).json()["keys"][0]["id"]
        assert c.delete(f"/api/v1/auth/keys/{kid}", headers=admin).status_code == 409  # the last admin key stays
        assert c.post("/v1/chat/completions", json=chat).status_code == 401
        c.app.state.keys.keys.clear()  # a table emptied behind the API's back still enforces
        assert c.post("/v1/chat/completions", json=chat).status_code == 401
        assert c.post("/api/v1/jobs", json={"kind": "inspect", "args": []}).status_code == 401
    (tmp_path / "keys.json").write_text("{}")
    with TestClient(create_app(service, api_key=KeyStore(tmp_path / "keys.json"))) as c:
        assert c.post("/v1/chat/completions", json=chat).status_code == 401
    with TestClient(create_app(service)) as c:  # no key, no key file: open
        assert c.post("/v1/chat/completions", json=chat).status_code == 200
    service.shutdown()


def test_job_listing_carries_no_log_text(tmp_path):
    from mfq_b200.server.jobs import Job
    log = tmp_path / "j.log"
    log.write_text("x" * 10000 + "END")
    job = Job("j", "inspect", ["inspect"], log)
    assert job.describe(0)["log_tail"] == ""
    assert job.describe(8)["log_tail"] == "xxxxxEND"

"""The HTTP contract is frozen: the application's schema equals the committed one, route by route."""

from mfq_b200.server import protocol


def test_schema_matches_the_committed_contract():
    now, frozen = protocol.current_schema(), protocol.frozen_schema()
    assert sorted(now["paths"]) == sorted(frozen["paths"]), "routes changed: regenerate with `python -m mfq_b200.server.protocol`"
    for path, item in frozen["paths"].items():
        assert sorted(item) == sorted(now["paths"][path]), path
        for method, op in item.items():
            got = now["paths"][path][method]
            assert [p["name"] for p in op.get("parameters", [])] == [p["name"] for p in got.get("parameters", [])], (path, method)
            assert sorted(op.get("responses", {})) == sorted(got.get("responses", {})), (path, method)
    assert now == frozen


def test_contract_covers_the_public_surfaces():
    paths = protocol.frozen_schema()["paths"]
    for needed in ("/v1/chat/completions", "/v1/messages", "/v1/models", "/api/v1/jobs", "/api/v1/catalog", "/api/v1/runtime/status",
                   "/api/v1/sessions", "/api/v1/auth/keys", "/metrics", "/health"):
        assert needed in paths, needed
    assert "post" in paths["/v1/chat/completions"] and "post" in paths["/api/v1/jobs"]
    from mfq_b200.server import ModelService, create_app
    ws = [r.path for r in create_app(ModelService()).routes if r.__class__.__name__ == "APIWebSocketRoute"]
    assert tuple(ws) == protocol.WEBSOCKET_ROUTES

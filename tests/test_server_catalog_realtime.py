"""Model catalog (discovery, aliases, persistence, routes), pool memory budgets, and the realtime WebSocket."""

import json

import numpy as np
import pytest
from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.catalog import ArtifactNotFound, ModelCatalog
from mfq_b200.server.pool import RuntimePool
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend


def _artifacts(root):
    from mfq_b200.cli import main
    (root / "packed").mkdir()
    assert main(["quantize", "synthetic:tiny-moe", str(root / "packed" / "tiny.mfq"), "--random-expert-mix", "NINT4,MXFP4"]) == 0
    hf = root / "hf-model"
    hf.mkdir()
    (hf / "config.json").write_text(json.dumps({"model_type": "llama"}))
    (hf / "model.safetensors").write_bytes(b"\0" * 64)
    (root / "other.gguf").write_bytes(b"GGUF" + b"\0" * 60)


def test_catalog_discovers_persists_and_resolves(tmp_path):
    _artifacts(tmp_path)
    state = tmp_path / "catalog.json"
    cat = ModelCatalog(state, roots=[tmp_path])
    rep = cat.scan()
    assert rep["entries"] == 3 and set(rep["added"]) == {"tiny", "hf-model", "other"}
    tiny = cat.resolve("tiny")
    assert tiny.kind == "mfq" and tiny.bytes > 0 and "MFE" in tiny.quantization["tensor_dtypes"]
    cat.alias("prod", "tiny")
    assert cat.resolve("prod").id == "tiny"
    with pytest.raises(ArtifactNotFound):
        cat.resolve("missing")
    again = ModelCatalog(state)  # restart: entries, roots and aliases come back
    assert again.resolve("prod").path == tiny.path and again.roots == cat.roots
    (tmp_path / "other.gguf").unlink()
    rep = again.scan()
    assert rep["removed"] == ["other"] and again.resolve("prod").id == "tiny"  # aliases survive a rescan


def test_catalog_routes(tmp_path):
    _artifacts(tmp_path)
    service = ModelService()
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    with TestClient(create_app(service, catalog=ModelCatalog(tmp_path / "c.json"))) as c:
        assert c.get("/api/v1/catalog").json()["models"] == []
        rep = c.post("/api/v1/catalog/scan", json={"roots": [str(tmp_path)]}).json()
        assert rep["entries"] == 3
        assert c.put("/api/v1/catalog/tiny/aliases/prod").json()["aliases"] == ["prod"]
        assert c.put("/api/v1/catalog/nope/aliases/x").status_code == 404
        ids = [m["id"] for m in c.get("/api/v1/catalog").json()["models"]]
        assert ids == ["hf-model", "other", "tiny"]
        assert c.delete("/api/v1/catalog/other").json()["removed"] is True
    service.shutdown()


class _Runtime:
    def __init__(self, name):
        self.name, self.kv = name, None

    def set_kv_budget(self, b):
        self.kv = b


def test_pool_memory_budget_evicts_rebalances_and_remembers_failures():
    now = [0.0]
    sizes = {"a": 40, "b": 30, "c": 50, "huge": 500, "broken": 0}
    loads = []

    def loader(name):
        loads.append(name)
        if name == "broken":
            raise OSError("cannot open")
        return _Runtime(name)
    pool = RuntimePool(loader, max_instances=4, max_memory_bytes=100, sizer=lambda n: sizes.get(n, 10), min_kv_bytes=5,
                       clock=lambda: now[0], load_failure_cooldown=30.0)
    a = pool.get("a")
    assert a.kv_budget_bytes == 60 and a.runtime.kv == 60  # everything the weights leave
    now[0] = 1.0
    b = pool.get("b")
    assert pool.rebalance() == {"a": 15, "b": 15} and a.runtime.kv == 15
    pool.configure("a", kv_share=2.0)
    assert pool.rebalance() == {"a": 20, "b": 10}
    now[0] = 2.0
    pool.get("c")  # 40 + 30 + 50 > 100: the least recently used idle model goes
    assert set(pool.instances) == {"b", "c"} and pool.evictions == 1
    with pytest.raises(MemoryError):
        pool.get("huge")
    with pytest.raises(OSError):
        pool.get("broken")
    with pytest.raises(OSError):
        pool.get("broken")  # inside the cool-down: the loader is not called again
    assert loads.count("broken") == 1
    now[0] = 40.0
    with pytest.raises(OSError):
        pool.get("broken")
    assert loads.count("broken") == 2
    pool.configure("b", idle_ttl=5.0)  # per-model idle time-out
    assert pool.reap() == ["b"]
    snap = pool.snapshot()
    assert snap["weight_bytes"] == 50 and snap["instances"][0]["kv_budget_bytes"] == 50


def test_realtime_socket_generates_pings_and_reports_errors():
    service = ModelService(max_queue=4, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    with TestClient(create_app(service)) as c:
        with c.websocket_connect("/api/v1/realtime") as ws:
            ws.send_text(json.dumps({"type": "ping"}))
            assert json.loads(ws.receive_text()) == {"type": "pong"}
            ws.send_text(json.dumps({"type": "generate", "id": "g1", "model": "echo", "messages": [{"role": "user", "content": "hi"}],
                                     "max_tokens": 8}))
            frames = []
            while not frames or frames[-1]["type"] not in ("done", "error"):
                frames.append(json.loads(ws.receive_text()))
            assert frames[0]["type"] == "started" and frames[0]["model"] == "echo"
            assert "".join(f["text"] for f in frames if f["type"] == "delta") == "ok!"
            assert frames[-1]["type"] == "done" and frames[-1]["text"] == "ok!" and frames[-1]["usage"]["completion_tokens"] == 3
            ws.send_text(json.dumps({"type": "generate", "id": "g2", "model": "nope", "messages": [{"role": "user", "content": "x"}]}))
            err = json.loads(ws.receive_text())
            assert err["type"] == "error" and err["id"] == "g2" and err["code"] == "model_not_found"
            ws.send_text("not json")
            assert json.loads(ws.receive_text())["code"] == "invalid_request"
            ws.send_text(json.dumps({"type": "cancel", "id": "unknown"}))
            assert json.loads(ws.receive_text())["code"] == "unknown_id"
    service.shutdown()


def test_realtime_socket_needs_an_inference_key():
    from starlette.websockets import WebSocketDisconnect
    service = ModelService()
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    with TestClient(create_app(service, api_key="secret")) as c:
        with pytest.raises(WebSocketDisconnect):
            with c.websocket_connect("/api/v1/realtime") as ws:
                ws.receive_text()
        with c.websocket_connect("/api/v1/realtime", headers={"authorization": "Bearer secret"}) as ws:
            ws.send_text(json.dumps({"type": "ping"}))
            assert json.loads(ws.receive_text())["type"] == "pong"
    service.shutdown()


def test_analysis_stats_and_purge_routes(tmp_path):
    _artifacts(tmp_path)
    service = ModelService()
    service.add_model("echo", EchoBackend(), ByteTokenizer())
    cat = ModelCatalog(tmp_path / "c.json", roots=[tmp_path])
    cat.scan()
    with TestClient(create_app(service, catalog=cat)) as c:
        r = c.get("/api/v1/catalog/tiny/analysis", params={"batch": 8, "context": 2048, "tensor_parallel": 2})
        assert r.status_code == 200
        doc = r.json()
        a = doc["analysis"]
        assert a["tensors"] > 10 and a["by_dtype"]["MFE"]["tensors"] == 6 and a["bytes"] == sum(v["bytes"] for v in a["by_dtype"].values())
        g = a["by_group"]["routed_experts"]
        assert g["weights"] == 2 * 8 * 3 * 256 * 128 and 4.0 < g["bits_per_weight"] < 5.2  # NINT4 / MXFP4 mix
        p = doc["parameters"]
        assert p["experts"] == 8 and p["top_k"] == 2 and p["active_per_token"] < p["total"]
        assert p["total"] - p["active_per_token"] == 2 * (8 - 2) * 3 * 256 * 128
        m = doc["memory"]
        assert m["gpus"] == 2 and m["per_gpu"]["total"] == sum(v for k, v in m["per_gpu"].items() if k != "total")
        # 16-token pages, (2 * 64 + 8) bytes per token, head and layer, one KV head per rank of two
        assert m["per_gpu"]["kv_cache"] == (8 * 128 + 1) * 2 * 1 * (2 * 64 + 8) * 16
        assert c.get("/api/v1/catalog/tiny/analysis", params={"batch": 0}).status_code == 400
        assert c.get("/api/v1/catalog/nope/analysis").status_code == 404
        hf = c.get("/api/v1/catalog/hf-model/analysis").json()
        assert hf["kind"] == "hf" and "analysis" not in hf
        # serving statistics: quantiles out of the histograms
        c.post("/v1/chat/completions", json={"model": "echo", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4})
        st = c.get("/api/v1/runtime/stats").json()["models"]["echo"]
        assert any(k.startswith("mfq_requests_total") or "request" in k for k in st["counters"])
        h = next(iter(st["histograms"].values()))
        assert h["count"] >= 1 and h["p50"] is not None and h["p95"] >= h["p50"]
        # purge deletes files below a root only
        gguf = tmp_path / "other.gguf"
        assert gguf.exists()
        r = c.delete("/api/v1/catalog/other", params={"purge": "true"})
        assert r.status_code == 200 and r.json()["purged"] and not gguf.exists()
        assert c.delete("/api/v1/catalog/other", params={"purge": "true"}).status_code == 404
        outside = tmp_path.parent / "outside.gguf"
        outside.write_bytes(b"GGUF" + b"\\0" * 8)
        try:
            from mfq_b200.server.catalog import Artifact
            cat.entries["outside"] = Artifact("outside", str(outside), "gguf", 12, 0.0)
            assert c.delete("/api/v1/catalog/outside", params={"purge": "true"}).status_code == 403 and outside.exists()
        finally:
            outside.unlink(missing_ok=True)


def test_identity_dataset_catalog_and_cache_profile_routes(tmp_path):
    import json

    from fastapi.testclient import TestClient

    from mfq_b200.calibration.dataset import build_text_corpus
    from mfq_b200.server import create_app
    from mfq_b200.server.catalog import ModelCatalog
    from mfq_b200.server.service import ModelService
    from mfq_b200.server.tokenizer import ByteTokenizer
    (tmp_path / "data").mkdir()
    records = [{"text": f"paragraph {i} " + "lorem ipsum dolor sit amet " * 12} for i in range(60)]
    build_text_corpus(ByteTokenizer(), tmp_path / "data" / "corpus-a", {"plain": records}, train_tokens=1024, validation_tokens=256,
                      sequence_length=64)
    (tmp_path / "data" / "other").mkdir()
    (tmp_path / "data" / "other" / "manifest.json").write_text(json.dumps({"format": "something-else"}))
    service = ModelService()
    with TestClient(create_app(service, catalog=ModelCatalog(roots=[tmp_path / "data"]))) as c:
        ident = c.get("/health/identity").json()
        assert ident["service"] == "mfq_b200" and len(ident["instance_id"]) == 32 and ident["models"] == []
        assert c.get("/health/identity").json()["instance_id"] == ident["instance_id"]
        cat = c.get("/api/v1/datasets/catalog").json()
        assert [d["name"] for d in cat["datasets"]] == ["corpus-a"]
        d = cat["datasets"][0]
        assert d["format"].startswith("mfq.calibration-corpus.") and d["sequence_length"] == 64 and d["tokens"]["train"] >= 1024
        assert c.get("/api/v1/models/none/cache-profile").status_code == 404
    service.shutdown()
    from mfq_b200.server.auth import required_scope
    assert required_scope("GET", "/health/identity") is None and required_scope("POST", "/api/v1/models/x/cache-profile") == "admin"


def test_cache_profile_route_reads_and_warms_an_expert_arena():
    import numpy as np
    from fastapi.testclient import TestClient

    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    from mfq_b200.server import create_app
    from mfq_b200.server.service import ModelService
    from mfq_b200.server.tokenizer import ByteTokenizer
    cfg = MoeDecoderConfig.tiny()
    tensors = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=4, std=0.05)
    model = MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu", expert_slots=3))
    res = model.residencies()
    assert res and all(r.slots == 3 for r in res)
    service = ModelService()
    service.add_model("moe", LLMEngine(model, max_batch=2, max_seq_len=64, device="cpu", use_graphs=False), ByteTokenizer())
    with TestClient(create_app(service)) as c:
        prof = c.get("/api/v1/models/moe/cache-profile").json()
        assert prof["model"] == "moe" and len(prof["layers"]) == len(res) and all(v["slots"] == 3 for v in prof["layers"].values())
        first = next(iter(prof["layers"]))
        prof["layers"][first]["heat"] = [0.0, 5.0, 0.0, 9.0, 1.0, 0.0, 0.0, 0.0]
        r = c.post("/api/v1/models/moe/cache-profile", json=prof).json()
        assert r == {"model": "moe", "warmed_experts": 3}
        assert sorted(int(e) for e in np.flatnonzero(res[0].slot_of >= 0)) == [1, 3, 4]
        prof["layers"][first]["heat"] = [1.0]
        assert c.post("/api/v1/models/moe/cache-profile", json=prof).json()["warmed_experts"] == 0   # a profile of another shape warms nothing
        assert c.post("/api/v1/models/moe/cache-profile", json={"layers": 3}).status_code == 400
    service.shutdown()

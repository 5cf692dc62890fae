"""Cluster routing (fake transport), hardware snapshot (fake NVML) and the cache control routes."""

import json
from types import SimpleNamespace

import pytest
from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.cluster import ClusterBackend, NoPeer
from mfq_b200.server.hardware import HardwareMonitor
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend


class FakeNet:
    """Two peers: ``a`` serves m1, ``b`` serves m1 and m2; either can be switched off or made to fail requests."""

    def __init__(self):
        self.models = {"http://a": ["m1"], "http://b": ["m1", "m2"]}
        self.down, self.fail_posts, self.calls = set(), set(), []

    def __call__(self, method, url, body, headers, stream):
        base, path = url[: url.index("/", 8)], url[url.index("/", 8):]
        self.calls.append((method, base, path))
        if base in self.down:
            raise ConnectionError(base)
        if path == "/health":
            return 200, {"status": "ok"}
        if path == "/v1/models":
            return 200, {"data": [{"id": m} for m in self.models[base]]}
        if base in self.fail_posts:
            return 502, {"error": {"code": "backend_failure"}}
        if stream:
            return 200, iter([b"data: {\"from\": \"%s\"}\n" % base.encode(), b"data: [DONE]\n"])
        return 200, {"served_by": base, "model": body["model"]}


def test_routing_spreads_load_and_skips_unhealthy_peers():
    now = [0.0]
    net = FakeNet()
    cl = ClusterBackend(["http://a", "http://b"], fetch=net, poll_interval=5.0, cooldown=15.0, clock=lambda: now[0])
    assert cl.models() == ["m1", "m2"]
    first = cl.forward("/v1/chat/completions", {"model": "m1"})[2]
    now[0] += 0.1
    second = cl.forward("/v1/chat/completions", {"model": "m1"})[2]
    assert {first, second} == {"http://a", "http://b"}  # least recently used peer goes next
    assert cl.forward("/v1/chat/completions", {"model": "m2"})[2] == "http://b"
    # a failing peer leaves the rotation, the request is retried on the other one
    net.fail_posts.add("http://a")
    now[0] += 1
    for _ in range(3):
        now[0] += 0.1
        status, out, url = cl.forward("/v1/chat/completions", {"model": "m1"})
        assert status == 200 and url == "http://b"
    assert [p["healthy"] for p in cl.status()] == [False, True]
    # after the cool-down it is probed again and comes back
    net.fail_posts.clear()
    now[0] += 20
    assert "http://a" in {cl.forward("/v1/chat/completions", {"model": "m1"})[2] for _ in range(2) if not now.__setitem__(0, now[0] + 0.1)}
    net.down.update({"http://a", "http://b"})
    now[0] += 20
    with pytest.raises(NoPeer):
        cl.forward("/v1/chat/completions", {"model": "m1"})


def test_server_forwards_models_it_does_not_hold():
    net = FakeNet()
    service = ModelService(max_queue=2, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    cluster = ClusterBackend(["http://a", "http://b"], fetch=net)
    with TestClient(create_app(service, cluster=cluster)) as c:
        ids = [m["id"] for m in c.get("/v1/models").json()["data"]]
        assert ids == ["echo", "m1", "m2"]
        r = c.post("/v1/chat/completions", json={"model": "m2", "messages": [{"role": "user", "content": "x"}]})
        assert r.status_code == 200 and r.json()["served_by"] == "http://b"
        with c.stream("POST", "/v1/chat/completions", json={"model": "m2", "stream": True, "messages": [{"role": "user", "content": "x"}]}) as r:
            lines = [l for l in r.iter_lines() if l]
        assert lines[0].startswith("data: ") and lines[-1] == "data: [DONE]"
        # local models never leave the box
        r = c.post("/v1/chat/completions", json={"model": "echo", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8})
        assert r.json()["choices"][0]["message"]["content"] == "ok!"
        assert len(c.get("/api/v1/cluster").json()["peers"]) == 2
    service.shutdown()


class FakeNvml:
    NVML_CLOCK_SM, NVML_TEMPERATURE_GPU = 1, 0

    def __init__(self):
        self.queries = 0

    def nvmlInit(self):
        pass

    def nvmlDeviceGetCount(self):
        return 2

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetName(self, h):
        return b"NVIDIA B200"

    def nvmlDeviceGetMemoryInfo(self, h):
        self.queries += 1
        return SimpleNamespace(total=180 << 30, used=(h + 1) << 30)

    def nvmlDeviceGetUtilizationRates(self, h):
        return SimpleNamespace(gpu=37)

    def nvmlDeviceGetClockInfo(self, h, kind):
        return 1965

    def nvmlDeviceGetPowerUsage(self, h):
        return 412000

    def nvmlDeviceGetTemperature(self, h, kind):
        raise RuntimeError("not supported")  # a missing query must not break the snapshot

    def nvmlDeviceGetCurrentClocksThrottleReasons(self, h):
        return 4


def test_hardware_snapshot_is_cached_and_read_only():
    now = [0.0]
    nv = FakeNvml()
    mon = HardwareMonitor(nvml=nv, ttl=1.0, clock=lambda: now[0])
    snap = mon.snapshot()
    assert [g["memory_used"] for g in snap["gpus"]] == [1 << 30, 2 << 30]
    assert snap["gpus"][0]["name"] == "NVIDIA B200" and snap["gpus"][0]["power_w"] == 412.0
    assert snap["gpus"][0]["temperature_c"] is None and snap["gpus"][1]["throttle_reasons"] == 4
    mon.snapshot()
    assert nv.queries == 2  # served from the cache
    now[0] += 1.5
    mon.snapshot()
    assert nv.queries == 4
    assert not [n for n in dir(nv) if "Set" in n or "Reset" in n]  # only getters are ever needed
    service = ModelService()
    with TestClient(create_app(service, hardware=mon)) as c:
        assert len(c.get("/api/v1/hardware").json()["gpus"]) == 2
        assert c.get("/api/v1/runtime/cache").json() == {"caches": []}
    service.shutdown()


def test_resource_history_keeps_a_bounded_timeline():
    from mfq_b200.server.hardware import ResourceHistory
    now = [0.0]
    mon = HardwareMonitor(nvml=FakeNvml(), ttl=0.0, clock=lambda: now[0])
    host = SimpleNamespace(cpu_percent=lambda interval=None: 12.5,
                           virtual_memory=lambda: SimpleNamespace(total=64 << 30, available=48 << 30))
    hist = ResourceHistory(mon, capacity=3, interval=0.01, host=host)
    for _ in range(5):
        now[0] += 1
        hist.sample()
    doc = hist.history()
    assert len(doc["samples"]) == 3 and doc["capacity"] == 3
    row = doc["samples"][-1]
    assert row["host"] == {"cpu_percent": 12.5, "memory_total": 64 << 30, "memory_used": 16 << 30}
    assert [g["memory_used"] for g in row["gpus"]] == [1 << 30, 2 << 30] and row["gpus"][0]["power_w"] == 412.0
    assert doc["peak"]["1"] == {"memory_used": 2 << 30, "utilization": 37, "power_w": 412.0}
    assert len(hist.history(last=2)["samples"]) == 2
    hist.start()  # the sampler thread adds rows by itself and stops on request
    import time as _t
    _t.sleep(0.08)
    hist.stop()
    assert hist._thread is None and len(hist.samples) == 3
    service = ModelService()
    with TestClient(create_app(service, hardware=mon)) as c:
        r = c.get("/api/v1/hardware/history", params={"last": 1}).json()
        assert len(r["samples"]) == 1 and len(r["samples"][0]["gpus"]) == 2
    service.shutdown()

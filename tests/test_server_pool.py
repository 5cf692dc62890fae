"""Runtime pool (LRU, slot gate error codes), session store, sampling profile resolution."""

import threading

import pytest

from mfq_b200.engine.scheduler import DeadlineExceeded, QueueFull, QueueTimeout
from mfq_b200.formats import runtime_profile as rp
from mfq_b200.server.pool import RuntimePool, SlotGate
from mfq_b200.server.sessions import SessionStore


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_pool_lru_eviction_and_idle_ttl():
    clock, loaded, dropped = Clock(), [], []
    pool = RuntimePool(lambda n: loaded.append(n) or f"rt-{n}", max_instances=2, idle_ttl=100.0, unloader=dropped.append, clock=clock)
    a = pool.get("a"); clock.t = 1; pool.get("b"); clock.t = 2; pool.get("a"); clock.t = 3
    pool.get("c")  # evicts b: least recently used
    assert dropped == ["rt-b"] and sorted(pool.instances) == ["a", "c"] and loaded == ["a", "b", "c"]
    assert a.gate.try_acquire()
    clock.t = 4
    pool.get("c")
    pool.get("d")  # a is busy, so c goes although a is older
    assert sorted(pool.instances) == ["a", "d"]
    assert not pool.unload("a")
    with pytest.raises(QueueFull):
        pool.instances["d"].gate.try_acquire()
        pool.get("e")
    pool.instances["d"].gate.release()
    a.gate.release()
    clock.t = 500
    assert sorted(pool.reap()) == ["a", "d"] and pool.snapshot()["instances"] == []


def test_slot_gate_codes_and_priority_order():
    clock = Clock()
    gate = SlotGate(concurrency=1, max_queue=2, clock=clock)
    gate.acquire()

    def fake_wait(cv, seconds):  # advance the clock instead of sleeping
        clock.t += seconds if seconds is not None else 1.0
    with pytest.raises(QueueTimeout):
        gate.acquire(queue_timeout=5.0, wait=fake_wait)
    with pytest.raises(DeadlineExceeded):
        gate.acquire(deadline=clock.t + 2.0, wait=fake_wait)
    assert gate.queued == 0 and gate.stats["timeouts"] == 1 and gate.stats["deadline"] == 1
    # two waiters: the high-priority one gets the slot first although it arrived second
    order, started = [], threading.Barrier(3)

    def waiter(tag, prio):
        started.wait()
        if tag == "high":
            while gate.queued < 1:
                pass
        gate.acquire(priority=prio)
        order.append(tag)
        gate.release()
    ts = [threading.Thread(target=waiter, args=("low", 0)), threading.Thread(target=waiter, args=("high", 5))]
    for t in ts:
        t.start()
    started.wait()
    while gate.queued < 2:
        pass
    with pytest.raises(QueueFull):
        gate.acquire()
    gate.release()
    for t in ts:
        t.join(5)
    assert order == ["high", "low"] and gate.stats["rejected_full"] == 1


def test_session_store(tmp_path):
    st = SessionStore(tmp_path / "s.db")
    s = st.create("first", model="m")
    assert st.append(s["id"], "user", "hi") == 0 and st.append(s["id"], "assistant", "hello", {"tokens": 2}) == 1
    other = st.create("second")
    st.append(other["id"], "user", "x")
    got = st.get(s["id"])
    assert [m["content"] for m in got["messages"]] == ["hi", "hello"] and got["messages"][1]["meta"] == {"tokens": 2}
    assert [r["title"] for r in st.list()] == ["second", "first"]
    assert st.rename(s["id"], "renamed") and st.list()[0]["title"] == "renamed"
    assert st.delete(other["id"]) and st.get(other["id"]) is None
    with pytest.raises(KeyError):
        st.append("nope", "user", "x")
    assert SessionStore(tmp_path / "s.db").get(s["id"])["title"] == "renamed"  # persisted


def test_sampling_profile_resolution():
    base = rp.resolve()
    assert base["source"] == "builtin" and base["chat"]["temperature"] == 0.0
    arch = rp.resolve(architecture="qwen3_next")
    assert arch["chat"]["top_k"] == 20 and arch["chat"]["enable_mtp"] and arch["source"].startswith("architecture-registry")
    assets = {"hf/generation_config.json": b'{"temperature": 0.3, "top_p": 0.5, "do_sample": true}'}
    hf = rp.resolve(assets=assets, architecture="qwen3_next")
    assert hf["chat"]["temperature"] == 0.3 and hf["chat"]["top_k"] == 20 and hf["source"] == "hf-generation-config"
    emb = rp.resolve({rp.HEADER_KEY: rp.make_profile({"temperature": 1.0, "mtp_max_draft_tokens": 5}, "test")}, assets, "qwen3_next")
    assert emb["chat"]["temperature"] == 1.0 and emb["chat"]["top_p"] == 0.5 and emb["source"] == "embedded"
    merged = rp.merge_request(emb["chat"], {"temperature": None, "top_p": 0.9, "bogus": 1})
    assert merged["temperature"] == 1.0 and merged["top_p"] == 0.9 and "bogus" not in merged
    with pytest.raises(ValueError):
        rp.make_profile({"nucleus": 1}, "x")
    with pytest.raises(ValueError):
        rp.validate({"schema": rp.SCHEMA, "version": 1, "chat": {"top_p": 1.5}})
    assert rp.from_generation_config('{"do_sample": false}')["chat"] == {"temperature": 0.0}

"""Expert residency (HBM slot arena in front of a host tier) on the CPU path: results equal the all-resident
computation, LRU/pinning bookkeeping, waves when a step needs more experts than slots, heat-driven rebalance."""

import torch

from mfq_b200.engine.expert_residency import ExpertResidency


def _fake_experts(n, h=8, i=4):
    g = torch.Generator().manual_seed(0)
    return (torch.randn((n, 2 * i, h), generator=g), torch.ones((n, 1, 1)), torch.randn((n, h, i), generator=g), torch.ones((n, 1, 1)))


def _ffn(x, ids, wt, gate_up, down):
    """Dense reference of a routed FFN over whichever expert table it is given (ids index that table; -1 skipped)."""
    out = torch.zeros_like(x)
    i = gate_up.shape[1] // 2
    for t in range(x.shape[0]):
        for k in range(ids.shape[1]):
            e = int(ids[t, k])
            if e < 0:
                continue
            gu = gate_up[e] @ x[t]
            out[t] += wt[t, k] * (down[e] @ (torch.nn.functional.silu(gu[:i]) * gu[i:]))
    return out


def test_residency_matches_all_resident_and_tracks_slots():
    n, slots = 10, 4
    gu, gus, dn, dns = _fake_experts(n)
    res = ExpertResidency(gu, gus, dn, dns, slots=slots, device="cpu")
    g = torch.Generator().manual_seed(1)
    x = torch.randn((6, 8), generator=g)
    ids = torch.tensor([[0, 1], [1, 2], [0, 2], [3, 1], [0, 3], [2, 3]], dtype=torch.int32)
    wt = torch.rand((6, 2), generator=g)
    want = _ffn(x, ids, wt, gu, dn)
    got = res.run(ids, lambda ids_slot, arena: _ffn(x, ids_slot, wt, arena.gate_up, arena.down))
    assert torch.allclose(got, want, atol=1e-6)
    assert res.stats["uploads"] == 4 and res.stats["waves"] == 1 and sorted(int(e) for e in (res.slot_of >= 0).nonzero()[0]) == [0, 1, 2, 3]
    # same experts again: all hits, no traffic
    res.run(ids, lambda ids_slot, arena: _ffn(x, ids_slot, wt, arena.gate_up, arena.down))
    assert res.stats["uploads"] == 4 and res.stats["hits"] == 4
    # a step that needs 6 distinct experts runs in two waves and still gives the all-resident answer
    ids2 = torch.tensor([[4, 5], [6, 7], [8, 9], [4, 9], [0, 5], [6, 1]], dtype=torch.int32)
    want2 = _ffn(x, ids2, wt, gu, dn)
    got2 = res.run(ids2, lambda ids_slot, arena: _ffn(x, ids_slot, wt, arena.gate_up, arena.down))
    assert torch.allclose(got2, want2, atol=1e-6) and res.stats["waves"] == 2 + 2 and res.stats["evictions"] >= 4
    assert (res.slot_of >= 0).sum() == slots and res.stats["upload_bytes"] == res.stats["uploads"] * res.bytes_per_expert


def test_rebalance_brings_hot_experts_in():
    n, slots = 8, 3
    res = ExpertResidency(*_fake_experts(n), slots=slots, device="cpu")
    res.run(torch.tensor([[0, 1], [2, 0]], dtype=torch.int32), lambda ids, arena: torch.zeros(1))
    res.heat[:] = [0.1, 0.2, 5.0, 9.0, 0.0, 7.0, 0.0, 0.0]  # 3 and 5 are hot but absent; 0 and 1 are cold residents
    swaps = res.rebalance(max_swaps=4)
    assert swaps == [(0, 3), (1, 5)]
    resident = sorted(int(e) for e in (res.slot_of >= 0).nonzero()[0])
    assert resident == [2, 3, 5]
    for e in resident:  # arena contents follow the book
        assert torch.equal(res.arena.gate_up[res.slot_of[e]], res.host[0][e])


def test_cache_profile_warms_a_fresh_arena(tmp_path):
    """Heat gathered by one run is saved; a fresh residency warmed from it starts with the hot experts resident."""
    from types import SimpleNamespace

    from mfq_b200.engine import moe_cache_profile as mcp
    n, slots = 10, 3

    def model():
        layers = []
        for _ in range(2):
            res = ExpertResidency(*_fake_experts(n), slots=slots, device="cpu")
            layers.append(SimpleNamespace(moe=SimpleNamespace(residency=res)))
        layers.insert(1, SimpleNamespace(moe=None))  # a dense layer in between
        return SimpleNamespace(w=SimpleNamespace(layers=layers, tp_rank=0))

    first = model()
    hot = torch.tensor([[7, 2], [7, 5], [7, 2], [2, 5]], dtype=torch.int32)
    for layer in (first.w.layers[0], first.w.layers[2]):
        for _ in range(3):
            layer.moe.residency.run(hot, lambda ids_slot, arena: torch.zeros(1))
    path = tmp_path / "profile.json"
    mcp.save(path, mcp.collect(first, "m"))
    doc = mcp.load(path)
    assert doc["format"] == mcp.FORMAT and set(doc["layers"]) == {"0", "2"} and doc["layers"]["0"]["heat"][7] > doc["layers"]["0"]["heat"][5] > 0
    fresh = model()
    assert mcp.apply(fresh, doc) == 6
    for layer in (fresh.w.layers[0], fresh.w.layers[2]):
        r = layer.moe.residency
        assert sorted(int(e) for e in (r.slot_of >= 0).nonzero()[0]) == [2, 5, 7] and r.stats["uploads"] == 3
        r.run(hot, lambda ids_slot, arena: torch.zeros(1))
        assert r.stats["uploads"] == 3 and r.stats["hits"] == 3  # first traffic: no upload at all
    # a profile of another model is ignored
    other = model()
    other.w.layers.pop()
    assert mcp.apply(other, doc) == 0 and mcp.load(tmp_path / "missing.json") is None


def test_optimistic_translate_counts_misses_and_settle_makes_the_step_whole():
    """Device-only translation: absent experts are skipped and counted; after ``settle`` the same step has no miss and
    equals the all-resident answer; a step with more distinct experts than slots asks for the wave path."""
    n, slots = 10, 4
    gu, gus, dn, dns = _fake_experts(n)
    res = ExpertResidency(gu, gus, dn, dns, slots=slots, device="cpu")
    miss = torch.zeros(1, dtype=torch.int32)
    res.enable_optimistic(miss)
    assert res.optimistic is False  # only the engine's decode step turns it on
    g = torch.Generator().manual_seed(2)
    x = torch.randn((4, 8), generator=g)
    wt = torch.rand((4, 2), generator=g)
    ids = torch.tensor([[0, 1], [1, 2], [-1, 2], [3, 1]], dtype=torch.int32)  # -1: an expert of another rank
    want = _ffn(x, ids, wt, gu, dn)

    def step():
        res.begin_step()
        miss.zero_()
        ids_slot = res.translate(ids)
        return ids_slot, _ffn(x, ids_slot, wt, res.arena.gate_up, res.arena.down)

    ids_slot, got = step()
    assert int(miss) == 7 and bool((ids_slot == -1).all()) and float(got.abs().max()) == 0.0  # cold arena: nothing ran
    assert res.step_hist.tolist()[:4] == [1, 3, 2, 1]
    assert res.settle() == "replay" and res.stats["uploads"] == 4
    ids_slot, got = step()
    assert int(miss) == 0 and torch.allclose(got, want, atol=1e-6)
    assert bool((ids_slot[2] == torch.tensor([-1, int(res.slot_of[2])])).all())
    assert res.settle() == "ok" and res.stats["uploads"] == 4 and res.stats["replays"] == 1
    # nothing stays pinned after a settle: a later step may evict any of them
    assert all(res.book.pins(e) == 0 for e in range(4)) if hasattr(res.book, "pins") else True
    wide = torch.tensor([[4, 5], [6, 7], [8, 9], [0, 1]], dtype=torch.int32)
    res.begin_step()
    miss.zero_()
    res.translate(wide)
    assert int(miss) == 6 and res.settle() == "fallback" and res.stats["fallbacks"] == 1
    # usage counted on the device reaches the host heat between steps
    before = res.heat.copy()
    res.absorb_heat()
    assert res.heat[1] > before[1] * res.decay and int(res.heat_dev.sum()) == 0


def test_cpu_decoder_with_an_arena_reads_the_host_tier():
    """On the CPU the fp32 path has no arena to manage: a model built with ``expert_slots`` gives the logits of the same
    model without it (the routed experts are read from the host tier, not from the uninitialised slot arena)."""
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    cfg = MoeDecoderConfig.tiny()
    tensors = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=4, std=0.05)
    prompts = [torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(1))]
    toks = []
    for slots in (None, 3):
        model = MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu", expert_slots=slots))
        assert bool(model.residencies()) == (slots is not None)
        toks.append(LLMEngine(model, max_batch=1, max_seq_len=48, device="cpu", use_graphs=False).generate(prompts, 6).tokens)
    assert torch.equal(toks[0], toks[1])

"""Layer placement across ranks (threads, CPU tensors): same logits as one rank, KV and weights only for local layers."""

import numpy as np
import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.llama import StepBuffers
from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
from mfq_b200.models.moe_lm import MoeConfig, init_weights
from mfq_b200.parallel.layer_parallel import plan_layers
from mfq_b200.parallel.local_collective import LocalGroup


def test_plan():
    assert plan_layers(8, 2) == [(0, 4), (4, 8)] and plan_layers(7, 3) in ([(0, 3), (3, 5), (5, 7)], [(0, 2), (2, 5), (5, 7)], [(0, 2), (2, 4), (4, 7)], [(0, 3), (3, 6), (6, 7)])
    assert plan_layers(8, 2, [3, 1]) == [(0, 6), (6, 8)]
    with pytest.raises(ValueError):
        plan_layers(2, 3)
    with pytest.raises(ValueError):
        plan_layers(8, 2, [1])


def _logits(cfg, model, prompt):
    eng = LLMEngine(model, max_batch=1, max_seq_len=96, device="cpu")
    n = prompt.numel()
    eng.cache.assign(0, 7, n)
    step = StepBuffers(input_ids=prompt.to(torch.int32), positions=torch.arange(n, dtype=torch.int32),
                       slots=eng.cache.slots(7, 0, n), cu_seqlens=[0, n])
    return model.forward(step, eng.cache, prefill=True).float(), eng


def test_placed_layers_give_the_single_rank_logits_exactly():
    base = MoeDecoderConfig.tiny()
    cfg = MoeDecoderConfig(**{**base.__dict__, "num_layers": 4})
    tensors = {k: v.numpy() for k, v in init_weights(MoeConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, num_experts=cfg.num_experts, top_k=cfg.top_k,
        moe_intermediate=cfg.moe_intermediate, shared_intermediate=cfg.shared_intermediate), seed=4, std=0.05).items()}
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(2))
    single, eng1 = _logits(cfg, MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu")), prompt)

    def rank(r, coll):
        w = MoeWeights.from_tensors(cfg, tensors, "cpu", lp_rank=r, lp_size=2, layer_split=[3, 1])
        model = MoeDecoderModel(cfg, w, collective=coll)
        out, eng = _logits(cfg, model, prompt)
        return out, sum(l is not None for l in w.layers), eng.cache.k.shape[0] if hasattr(eng.cache, "k") else model.local_layers

    results = LocalGroup(2).run(rank)
    for out, _held, _kv in results:
        assert torch.equal(out, single)  # the same arithmetic in the same order: bit-identical
    assert [r[1] for r in results] == [3, 1]
    with pytest.raises(ValueError, match="mutually exclusive"):
        MoeWeights.from_tensors(cfg, tensors, "cpu", 0, 2, lp_rank=0, lp_size=2)


def test_generation_through_the_engine_matches():
    cfg = MoeDecoderConfig.tiny()
    tensors = {k: v.numpy() for k, v in init_weights(MoeConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, num_experts=cfg.num_experts, top_k=cfg.top_k,
        moe_intermediate=cfg.moe_intermediate, shared_intermediate=cfg.shared_intermediate), seed=5, std=0.05).items()}
    prompt = torch.arange(5, 25)
    want = LLMEngine(MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu")), max_batch=1, max_seq_len=64, device="cpu").generate([prompt], 6).tokens

    def rank(r, coll):
        model = MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu", lp_rank=r, lp_size=2), collective=coll)
        eng = LLMEngine(model, max_batch=1, max_seq_len=64, device="cpu")
        assert model.local_layers == cfg.num_layers // 2
        return eng.generate([prompt], 6).tokens

    for got in LocalGroup(2).run(rank):
        assert torch.equal(got, want)

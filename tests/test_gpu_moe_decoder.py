"""FP8 MoE decoder on the GPU kernels against its CPU reference path, and graph decode."""

import copy
import dataclasses

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.evaluation.kld import compare_logits
from mfq_b200.models.llama import StepBuffers
from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
from mfq_b200.models.moe_lm import MoeConfig, init_weights, quantize_moe_checkpoint
from gpu_common import check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def test_moe_decoder_gpu_matches_cpu_and_graphs():
    require_gpu_lib()
    cfg = MoeDecoderConfig.tiny()
    ck = quantize_moe_checkpoint(init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128,
                                                        shared_intermediate=128), seed=9, std=0.05), "NINT4,NVQ3,MXFP4")
    prompt = torch.randint(0, cfg.vocab_size, (50,), generator=torch.Generator().manual_seed(2))
    outs = {}
    for dev in ("cpu", "cuda"):
        model = MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, ck, dev))
        eng = LLMEngine(model, max_batch=2, max_seq_len=96, device=dev, use_graphs=False)
        eng.cache.assign(0, 0, 50)
        step = StepBuffers(input_ids=prompt.to(dev, torch.int32), positions=torch.arange(50, dtype=torch.int32, device=dev),
                           slots=eng.cache.slots(0, 0, 50).to(dev), cu_seqlens=[0, 50])
        outs[dev] = model.forward(step, eng.cache, prefill=True).float().cpu()
    check_status()
    r = compare_logits(outs["cpu"], outs["cuda"])
    assert r.kld < 0.01 and r.top1_agreement > 0.8, r
    model = MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, ck, "cuda"))
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (17, 40)]
    a = LLMEngine(model, max_batch=2, max_seq_len=96, use_graphs=False).generate(prompts, 8)
    b = LLMEngine(model, max_batch=2, max_seq_len=96, use_graphs=True).generate(prompts, 8)
    assert torch.equal(a.tokens, b.tokens)
    check_status()


def test_host_tier_experts_match_all_resident():
    """Experts behind a 3-slot HBM arena (uploads on demand, waves when a step needs more) give the same logits."""
    import torch
    from gpu_common import check_status, require_gpu_lib
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import StepBuffers
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    require_gpu_lib()
    cfg = MoeDecoderConfig.tiny()
    tensors = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=4, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(3))

    def logits(weights):
        eng = LLMEngine(MoeDecoderModel(cfg, weights), max_batch=2, max_seq_len=64, use_graphs=False)
        eng.cache.assign(0, 1, 24)
        step = StepBuffers(input_ids=prompt.cuda().int(), positions=torch.arange(24, dtype=torch.int32, device="cuda"),
                           slots=eng.cache.slots(1, 0, 24).cuda(), cu_seqlens=[0, 24])
        return eng.model.forward(step, eng.cache, prefill=True).float().cpu()

    full = logits(MoeWeights.from_tensors(cfg, tensors, "cuda"))
    tiered_w = MoeWeights.from_tensors(cfg, tensors, "cuda", expert_slots=3)
    tiered = logits(tiered_w)
    check_status()
    res = tiered_w.layers[0].moe.residency
    assert res is not None and res.stats["uploads"] >= 3 and res.stats["waves"] >= 2  # 8 experts, 3 slots
    scale = float(full.abs().max())
    err = (full - tiered).abs()
    # same FP8 experts; the waves round their partial sums to bf16 separately, which can flip a later layer's routing
    assert float(err.mean()) <= 0.02 * scale and float(err.max(-1).values.median()) <= 0.1 * scale


@pytest.mark.parametrize("slots", [5, 3])
def test_expert_residency_under_graphs_replays_misses(slots):
    """An expert arena of ``slots`` of 8 experts decoding inside CUDA graphs: ids are translated on the device, a step
    that met an absent expert is run again after the upload (or in waves when it needs more experts than slots), and
    the tokens equal the eager wave-by-wave engine's."""
    import torch
    from gpu_common import check_status, require_gpu_lib
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    require_gpu_lib()
    cfg = MoeDecoderConfig.tiny()
    tensors = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=4, std=0.05)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (17, 40)]

    eager = LLMEngine(MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cuda", expert_slots=slots)),
                      max_batch=2, max_seq_len=96, use_graphs=False)
    want = eager.generate(prompts, 12).tokens
    eng = LLMEngine(MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cuda", expert_slots=slots)),
                    max_batch=2, max_seq_len=96, use_graphs=True)
    assert eng.enable_expert_residency_graphs()
    got = eng.generate(prompts, 12).tokens
    check_status()
    assert torch.equal(got, want)
    st = eng.residency_stats
    assert st["steps"] >= 11 and len(eng.graphs) >= 1
    assert st["replays"] + st["fallbacks"] < st["steps"] * eng.residency_replays  # most steps ran once, from the graph
    res = eng.model.residencies()
    assert all(not r.optimistic for r in res) and sum(r.stats["uploads"] for r in res) >= slots


def test_probability_scores_match_the_cpu_engine():
    """`LLMEngine.score` (chunked prefill with logits at the scored positions only) on the GPU against the fp32 CPU path."""
    import torch
    from gpu_common import check_status, require_gpu_lib
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    require_gpu_lib()
    cfg = MoeDecoderConfig.tiny()
    tensors = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=6, std=0.05)
    ids = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(8)).tolist()
    scores = {}
    for dev in ("cpu", "cuda"):
        eng = LLMEngine(MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, dev)), max_batch=2, max_seq_len=128, device=dev, use_graphs=False)
        eng.prefill_chunk = 32                     # three chunks, the scored span starts inside the second
        scores[dev] = torch.tensor(eng.score(1, ids, 40))
        assert 1 not in eng.row_seq
    check_status()
    assert scores["cuda"].shape == (30,) and bool((scores["cuda"] <= 0).all())
    # FP8 weights and activations on one side, fp32 on the other, at log-probabilities around -7
    assert float((scores["cuda"] - scores["cpu"]).abs().max()) < 0.4 and float((scores["cuda"] - scores["cpu"]).abs().mean()) < 0.1

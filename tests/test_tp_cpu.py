"""Tensor / expert parallel model code on the CPU: in-process ranks (threads) against the single-rank result."""

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights, kv_head_rows
from mfq_b200.parallel.local_collective import LocalGroup


def test_local_collective_primitives():
    g = LocalGroup(4)

    def body(rank, c):
        h = torch.ones(2, 3)
        c.allreduce_rows(torch.full((2, 3), float(rank)), h)
        cols = c.gather_columns(torch.full((2, 1), float(rank)))
        logits = torch.zeros(2, 5)
        logits[0, 2] = 7.0 if rank == 3 else 1.0       # row 0: rank 3 wins
        logits[1, 1] = 5.0 if rank in (1, 2) else 0.0  # row 1: tie between ranks 1 and 2 -> lowest global index
        return h, cols, c.argmax(logits)

    for h, cols, am in g.run(body):
        assert torch.equal(h, torch.full((2, 3), 7.0))  # 1 + 0 + 1 + 2 + 3
        assert cols.tolist() == [[0, 1, 2, 3], [0, 1, 2, 3]]
        assert am.tolist() == [3 * 5 + 2, 1 * 5 + 1]


def test_a_failing_rank_does_not_hang_the_others():
    def body(rank, c):
        if rank == 1:
            raise ValueError("rank 1 fails before the collective")
        c.barrier()
    with pytest.raises(ValueError):
        LocalGroup(3, timeout=10.0).run(body)


def test_kv_head_rows_replicates_when_ranks_outnumber_heads():
    w = torch.arange(2 * 4 * 3, dtype=torch.float32).reshape(8, 3)  # 2 heads of 4 rows
    assert torch.equal(kv_head_rows(w, 2, 4, 1, 2), w[4:8])
    got = [kv_head_rows(w, 2, 4, r, 4) for r in range(4)]
    assert torch.equal(got[0], w[:4]) and torch.equal(got[1], w[:4]) and torch.equal(got[2], w[4:]) and torch.equal(got[3], w[4:])
    with pytest.raises(ValueError):
        kv_head_rows(w, 2, 4, 0, 3)


def _prefill_logits(cfg, model, prompt):
    from mfq_b200.models.llama import StepBuffers
    eng = LLMEngine(model, max_batch=1, max_seq_len=96, device="cpu")
    n = prompt.numel()
    eng.cache.assign(0, 7, n)
    if eng.rec_state is not None:
        eng.rec_state.reset(0)
    step = StepBuffers(input_ids=prompt.to(torch.int32), positions=torch.arange(n, dtype=torch.int32),
                       slots=eng.cache.slots(7, 0, n), cu_seqlens=[0, n],
                       state_slots=eng.row_ids[:1] if eng.rec_state is not None else None)
    return model.forward(step, eng.cache, prefill=True).float()


def _check_parallel(cfg, build, world, prompt, tol, min_cos=0.97, min_row_cos=0.99):
    single = _prefill_logits(cfg, build(0, 1, None), prompt)
    ranks = LocalGroup(world).run(lambda rank, coll: _prefill_logits(cfg, build(rank, world, coll), prompt))
    for r in ranks[1:]:
        assert torch.equal(r, ranks[0])  # every rank ends with the same gathered logits
    assert ranks[0].shape == single.shape
    err = (ranks[0] - single).abs()
    scale = float(single.abs().max())
    # row-parallel inputs are quantized per shard instead of per full row, so FP8 rounding falls differently: the
    # logits agree to quantization noise (a wrong shard or head mapping would decorrelate them completely)
    # (a token whose expert choice flips under that noise moves its whole row, so rows are judged by their median)
    cos = float(torch.nn.functional.cosine_similarity(ranks[0].flatten(), single.flatten(), dim=0))
    row_cos = float(torch.nn.functional.cosine_similarity(ranks[0], single, dim=1).median())
    assert cos > min_cos and row_cos > min_row_cos and float(err.mean()) <= tol * scale, (cos, row_cos, float(err.mean()), float(err.max()), scale)


@pytest.mark.parametrize("world", [2, 4])
def test_llama_tensor_parallel_matches_single_rank(world):
    """TP = 4 on 2 KV heads replicates each head on two ranks."""
    cfg = LlamaConfig.tiny()
    prompt = torch.randint(0, cfg.vocab_size, (33,), generator=torch.Generator().manual_seed(33))
    build = lambda rank, w, coll: LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=3, std=0.05, tp_rank=rank, tp_size=w), collective=coll)
    _check_parallel(cfg, build, world, prompt, tol=0.03)


def test_moe_decoder_expert_parallel_matches_single_rank():
    """Experts split over the ranks (each adds the partial of its own experts), attention tensor-parallel, shared expert
    too narrow to shard -> rank 0 carries it."""
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    cfg = MoeDecoderConfig.tiny()
    tensors = {k: v.numpy() for k, v in init_weights(MoeConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, num_experts=cfg.num_experts, top_k=cfg.top_k,
        moe_intermediate=cfg.moe_intermediate, shared_intermediate=cfg.shared_intermediate), seed=4, std=0.05).items()}
    prompt = torch.randint(0, cfg.vocab_size, (29,), generator=torch.Generator().manual_seed(2))
    build = lambda rank, w, coll: MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu", rank, w), collective=coll)
    _check_parallel(cfg, build, 2, prompt, tol=0.03)


def test_hybrid_tensor_parallel_matches_single_rank():
    """Gated DeltaNet heads, attention heads and experts all split over two ranks."""
    from mfq_b200.models.hybrid import HybridConfig, HybridModel, HybridWeights, init_hybrid_weights
    cfg = HybridConfig.tiny()
    tensors = init_hybrid_weights(cfg, seed=3, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (27,), generator=torch.Generator().manual_seed(5))
    build = lambda rank, w, coll: HybridModel(cfg, HybridWeights.from_tensors(cfg, tensors, "cpu", rank, w), collective=coll)
    # four MoE layers and the recurrent state amplify the rounding noise (and flip a few expert choices); a wrong head
    # or shard mapping lands near 0.3
    _check_parallel(cfg, build, 2, prompt, tol=0.05, min_cos=0.95, min_row_cos=0.97)


def test_random_hybrid_weights_are_shards_of_one_model():
    """The random-init builder used by the benchmark: every rank draws only its experts, yet TP = 2 is the same model
    as TP = 1 (also with the MTP head's block)."""
    from mfq_b200.models.hybrid import HybridConfig, HybridModel, random_hybrid_weights
    cfg = HybridConfig.tiny()
    one = random_hybrid_weights(cfg, "cpu", seed=2, std=0.05, mtp=True, expert_chunk=3)
    two = [random_hybrid_weights(cfg, "cpu", seed=2, std=0.05, mtp=True, expert_chunk=3, tp_rank=r, tp_size=2) for r in range(2)]
    full = one.layers[0].moe.gate_up
    assert torch.equal(torch.cat([t.layers[0].moe.gate_up for t in two]).view(torch.uint8), full.view(torch.uint8))
    assert two[1].layers[0].moe.e_lo == cfg.num_experts // 2 and torch.equal(two[0].embed, one.embed)
    assert torch.equal(torch.cat([t.mtp.layer.moe.down for t in two]).view(torch.uint8), one.mtp.layer.moe.down.view(torch.uint8))
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(8))
    build = lambda rank, w, coll: HybridModel(cfg, one if w == 1 else two[rank], collective=coll)
    _check_parallel(cfg, build, 2, prompt, tol=0.05, min_cos=0.95, min_row_cos=0.97)

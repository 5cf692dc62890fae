"""Prefix cache in the engine (CPU path): cached leading blocks are restored into KV pages instead of recomputed."""

import torch

from mfq_b200 import native
from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights


def test_prefix_blocks_are_reused_and_results_unchanged(tmp_path):
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=2, std=0.05)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, cfg.vocab_size, (70,), generator=g)
    p1 = torch.cat([shared, torch.randint(0, cfg.vocab_size, (9,), generator=g)])
    p2 = torch.cat([shared, torch.randint(0, cfg.vocab_size, (14,), generator=g)])
    plain = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=128, device="cpu")
    want1 = plain.generate([p1], 5).tokens[0].tolist()
    plain.release(0)
    want2 = plain.generate([p2], 5).tokens[0].tolist()
    pc = native.PrefixCache(tmp_path / "kv", ram_budget=64 << 20, disk_budget=64 << 20, block_tokens=32)
    eng = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=128, device="cpu", prefix_cache=pc, prefix_salt="tiny-llama/seed2")
    assert eng.generate([p1], 5).tokens[0].tolist() == want1
    assert eng.prefix_stats == {"lookups": 1, "blocks_hit": 0, "blocks_stored": 2, "tokens_skipped": 0}
    eng.release(0)
    # same 64-token prefix (2 blocks), different tail: both blocks come from the cache, the answer does not change
    assert eng.generate([p2], 5).tokens[0].tolist() == want2
    assert eng.prefix_stats["blocks_hit"] == 2 and eng.prefix_stats["tokens_skipped"] == 64
    eng.release(0)
    # a fresh engine (e.g. after a restart) finds the blocks in the file tier
    pc.flush()
    pc.close()
    pc2 = native.PrefixCache(tmp_path / "kv", ram_budget=64 << 20, disk_budget=64 << 20, block_tokens=32)
    eng2 = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=128, device="cpu", prefix_cache=pc2, prefix_salt="tiny-llama/seed2")
    assert eng2.generate([p1], 5).tokens[0].tolist() == want1 and eng2.prefix_stats["blocks_hit"] == 2
    # another model (salt) never sees these blocks
    eng3 = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=128, device="cpu", prefix_cache=pc2, prefix_salt="other")
    eng3.generate([p1], 2)
    assert eng3.prefix_stats["blocks_hit"] == 0
    pc2.close()

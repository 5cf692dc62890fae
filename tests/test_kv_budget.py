"""KV budget planning."""

import pytest

from mfq_b200.engine import kv_budget as kb


def test_page_cost_and_plan():
    pb = kb.page_bytes(layers=32, kv_heads=8, head_dim=128)
    assert pb == 32 * 8 * (256 + 8) * 16
    full = kb.plan(budget_bytes=1 << 40, layers=32, kv_heads=8, head_dim=128, max_batch=64, max_seq_len=4096)
    assert full.num_pages == 64 * 256 + 1 and not full.oversubscribed
    tight = kb.plan(budget_bytes=4 << 30, layers=32, kv_heads=8, head_dim=128, max_batch=64, max_seq_len=4096)
    assert tight.oversubscribed and tight.kv_bytes <= 4 << 30 and tight.num_pages >= 257
    with pytest.raises(MemoryError):
        kb.plan(budget_bytes=64 << 20, layers=32, kv_heads=8, head_dim=128, max_batch=64, max_seq_len=4096)
    hybrid = kb.plan(budget_bytes=8 << 30, layers=12, kv_heads=2, head_dim=256, max_batch=64, max_seq_len=4096,
                     state_bytes_per_row=36 * 32 * 128 * 128 * 4)
    assert hybrid.state_bytes == 64 * 36 * 32 * 128 * 128 * 4 and hybrid.kv_bytes + hybrid.state_bytes <= 8 << 30


def test_engine_with_a_small_pool_still_serves(tmp_path):
    import torch
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    model = LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=1, std=0.05))
    p = kb.plan(budget_bytes=kb.page_bytes(cfg.num_layers, model.hk, cfg.head_dim) * 12, layers=cfg.num_layers, kv_heads=model.hk,
                head_dim=cfg.head_dim, max_batch=4, max_seq_len=128)
    assert p.num_pages == 12 and p.oversubscribed
    eng = LLMEngine(model, max_batch=4, max_seq_len=128, device="cpu", num_pages=p.num_pages)
    out = eng.generate([torch.randint(0, cfg.vocab_size, (20,))], 4)
    assert out.tokens.shape == (1, 4)

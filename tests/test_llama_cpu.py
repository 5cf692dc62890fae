"""CPU path of the FP8 Llama: decode must agree with re-running the grown prompt through prefill."""

import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights


def test_decode_consistent_with_prefill():
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=5, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(0))
    eng = LLMEngine(LlamaModel(cfg, w), max_batch=1, max_seq_len=64, device="cpu")
    gen = eng.generate([prompt], 6).tokens[0]
    for t in range(1, 6):
        eng2 = LLMEngine(LlamaModel(cfg, w), max_batch=1, max_seq_len=64, device="cpu")
        grown = torch.cat([prompt, gen[:t].long()])
        assert int(eng2.prefill(0, grown)) == int(gen[t]), f"token {t} differs between decode and prefill"


def test_kv_pages_are_released():
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=5)
    eng = LLMEngine(LlamaModel(cfg, w), max_batch=1, max_seq_len=64, device="cpu")
    free0 = eng.cache.allocator.free_pages
    eng.prefill(0, torch.arange(20))
    assert eng.cache.allocator.free_pages < free0
    eng.prefill(0, torch.arange(5))
    assert eng.cache.allocator.free_pages == free0 - 1


def test_w4_weights_decode_consistent_with_prefill():
    """The 4-bit weight path (CPU reference of the in-pipeline-decode GEMM): a decode step continues the prefill."""
    import torch
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights, W4Linear
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=1, std=0.05, weight_format="w4")
    assert isinstance(w.layers[0].qkv, W4Linear) and w.layers[0].qkv.w.bits_per_weight <= 5.01
    eng = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=64, device="cpu")
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(0))
    first = eng.prefill(0, prompt)
    eng.grow(0, 32)
    eng.active.zero_()
    eng.active[0] = 1
    eng.decode_step(1)
    second = int(eng.sampled[0])
    assert eng.prefill(1, torch.cat([prompt, torch.tensor([first])])) == second


def test_chunked_prefill_equals_one_shot_prefill():
    """A prompt prefilled in chunks (each chunk attends to the cached past) predicts what the one-shot prefill predicts,
    and decoding continues identically."""
    import torch
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=2, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (45,), generator=torch.Generator().manual_seed(3))
    whole = LLMEngine(LlamaModel(cfg, w), max_batch=1, max_seq_len=96, device="cpu")
    parts = LLMEngine(LlamaModel(cfg, w), max_batch=1, max_seq_len=96, device="cpu", prefill_chunk=16)
    a = whole.generate([prompt], 6).tokens[0].tolist()
    b = parts.generate([prompt], 6).tokens[0].tolist()
    assert a == b

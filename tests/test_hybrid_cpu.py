"""Hybrid (Gated DeltaNet + gated attention + MoE) model on the CPU reference path."""

import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.hybrid import HybridConfig, HybridModel, HybridWeights, init_hybrid_weights
from mfq_b200.models.llama import StepBuffers


def _engine(max_batch=2):
    cfg = HybridConfig.tiny()
    w = HybridWeights.from_tensors(cfg, init_hybrid_weights(cfg, seed=3, std=0.05), "cpu")
    return cfg, LLMEngine(HybridModel(cfg, w), max_batch=max_batch, max_seq_len=64, device="cpu")


def test_layer_pattern_and_weights():
    cfg = HybridConfig.tiny()
    assert [cfg.is_linear(i) for i in range(4)] == [True, False, True, False]
    w = HybridWeights.from_tensors(cfg, init_hybrid_weights(cfg, seed=3), "cpu")
    assert w.layers[0].gdn is not None and w.layers[0].qkv is None
    assert w.layers[1].gdn is None and w.layers[1].gated and w.layers[1].q_norm.shape == (128,)
    # q | k | v | z | b | a rows of the stacked projection
    assert w.layers[0].gdn.in_proj.q.shape[0] == cfg.conv_dim + 4 * 128 + 2 * 4


def test_decode_continues_prefill_exactly_like_a_longer_prefill():
    """Recurrent state + KV after prefill(n) and one decode step must predict what prefill(n + 1) predicts."""
    cfg, eng = _engine()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (13,), generator=g)
    first = eng.prefill(0, prompt)
    eng.grow(0, 32)
    eng.active.zero_()
    eng.active[0] = 1
    eng.decode_step(1)
    second = int(eng.sampled[0])
    eng.release(0)
    longer = torch.cat([prompt, torch.tensor([first])])
    assert eng.prefill(1, longer) == second


def test_rows_do_not_disturb_each_other():
    cfg, eng = _engine()
    g = torch.Generator().manual_seed(1)
    p0, p1 = (torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (9, 17))
    solo = eng.generate([p0], 6).tokens[0].tolist()
    eng.release(0)
    both = eng.generate([p0, p1], 6).tokens
    assert both[0].tolist() == solo


def _with_mtp_head(cfg, w, seed=9):
    """Attach a random MTP head (dense attention block) to hybrid weights."""
    from mfq_b200.models.llama import LlamaWeights, MtpHead
    donor = LlamaWeights.random_init(cfg, "cpu", seed=seed, std=0.05, mtp=True)
    w.mtp = donor.mtp
    return w


def test_mtp_cycles_on_hybrid_model_are_lossless():
    """Verify windows checkpoint the recurrent state per token and commit the accepted prefix: the tokens must be
    the ones plain greedy decoding produces."""
    cfg = HybridConfig.tiny()
    w = _with_mtp_head(cfg, HybridWeights.from_tensors(cfg, init_hybrid_weights(cfg, seed=3, std=0.05), "cpu"))
    eng = LLMEngine(HybridModel(cfg, w), max_batch=2, max_seq_len=96, device="cpu", mtp_draft_tokens=2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (9, 14)]
    plain = eng.generate(prompts, 10).tokens
    for r in range(2):
        eng.release(r)
    spec = eng.generate(prompts, 10, use_mtp=True).tokens
    for r in range(2):
        a, b = plain[r].tolist(), spec[r].tolist()
        n = 0
        while n < len(a) and a[n] == b[n]:
            n += 1
        assert n >= 8, (a, b)  # float summation order may flip a near-tie late in the sequence
    # oracle drafts: all accepted, state committed at the last window position
    for r in range(2):
        eng.release(r)
    truth = plain[0].tolist()
    eng.prefill(0, prompts[0])
    eng.grow(0, 40)
    eng.draft[0] = torch.tensor(truth[1:3], dtype=torch.int32)
    eng.active.zero_()
    eng.active[0] = 1
    eng.mtp_step(1)
    n = int(eng.n_out[0])
    assert n >= 2 and eng.out_tokens[0, :n].tolist() == truth[1 : 1 + n]
    # and decoding on from the committed state still follows the plain sequence
    eng.decode_step(1)
    assert int(eng.sampled[0]) == truth[1 + n]


def test_hybrid_chunked_prefill_carries_recurrent_state():
    cfg = HybridConfig.tiny()
    w = HybridWeights.from_tensors(cfg, init_hybrid_weights(cfg, seed=3, std=0.05), "cpu")
    prompt = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(5))
    whole = LLMEngine(HybridModel(cfg, w), max_batch=1, max_seq_len=96, device="cpu")
    parts = LLMEngine(HybridModel(cfg, w), max_batch=1, max_seq_len=96, device="cpu", prefill_chunk=16)
    assert whole.generate([prompt], 5).tokens[0].tolist() == parts.generate([prompt], 5).tokens[0].tolist()

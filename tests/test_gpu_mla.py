"""Latent attention model on the GPU kernels (256-wide padded heads) against the CPU reference path."""

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.llama import StepBuffers
from mfq_b200.models.mla import MlaConfig, MlaModel, random_mla_weights
from gpu_common import check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def _to(weights, dev):
    """Move a weight tree to ``dev`` (the builder draws from a device generator, so build once on the CPU and copy)."""
    import copy
    import dataclasses

    def move(x):
        if isinstance(x, torch.Tensor):
            return x.to(dev)
        if isinstance(x, list):
            return [move(v) for v in x]
        if dataclasses.is_dataclass(x) and not isinstance(x, type):
            y = copy.copy(x)
            for f in dataclasses.fields(x):
                setattr(y, f.name, move(getattr(x, f.name)))
            return y
        return x
    return move(weights)


def _logits(eng, prompt, dev):
    n = prompt.numel()
    eng.cache.assign(0, 555, n)
    step = StepBuffers(input_ids=prompt.to(dev, torch.int32), positions=torch.arange(n, dtype=torch.int32, device=dev),
                       slots=eng.cache.slots(555, 0, n).to(dev), cu_seqlens=[0, n])
    out = eng.model.forward(step, eng.cache, prefill=True).float().cpu()
    eng.cache.release(555)
    return out


def test_mla_attention_alone_matches_cpu_tightly():
    """All layers dense: no routing decisions that rounding could flip, so the latent-attention path itself is compared."""
    import dataclasses
    require_gpu_lib()
    cfg = dataclasses.replace(MlaConfig.tiny(), first_dense_layers=3)
    w_cpu = random_mla_weights(cfg, "cpu", seed=4, std=0.05, expert_chunk=3)
    gpu = LLMEngine(MlaModel(cfg, _to(w_cpu, "cuda")), max_batch=2, max_seq_len=128)
    cpu = LLMEngine(MlaModel(cfg, w_cpu), max_batch=2, max_seq_len=128, device="cpu")
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(3))
    lg, lc = _logits(gpu, prompt, "cuda"), _logits(cpu, prompt, "cpu")
    check_status()
    scale = float(lc.abs().max())
    cos = float(torch.nn.functional.cosine_similarity(lg.flatten(), lc.flatten(), dim=0))
    # measured: cosine 0.9954, mean error 1.7 % of the logit range -- the FP8 rounding level of a three-layer model
    assert cos > 0.99 and float((lg - lc).abs().mean()) <= 0.03 * scale, (cos, float((lg - lc).abs().mean()), scale)


def test_mla_gpu_matches_cpu_and_graph_decode():
    require_gpu_lib()
    cfg = MlaConfig.tiny()
    w_cpu = random_mla_weights(cfg, "cpu", seed=1, std=0.05, expert_chunk=3)
    gpu = LLMEngine(MlaModel(cfg, _to(w_cpu, "cuda")), max_batch=4, max_seq_len=128)
    cpu = LLMEngine(MlaModel(cfg, w_cpu), max_batch=4, max_seq_len=128, device="cpu")
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(2))
    lg, lc = _logits(gpu, prompt, "cuda"), _logits(cpu, prompt, "cpu")
    check_status()
    scale = float(lc.abs().max())
    err = (lg - lc).abs()
    # a token whose expert choice flips under FP8 rounding moves its whole logit row: bound the typical row tightly
    # (sigmoid scores with a 2.5x routed scale make this tiny model more sensitive than the softmax ones)
    cos = float(torch.nn.functional.cosine_similarity(lg.flatten(), lc.flatten(), dim=0))
    assert float(err[0].max()) <= 0.02 * scale  # the first token attends to itself only: no flips, kernels must agree
    assert cos > 0.95 and float(err.mean()) <= 0.06 * scale and float(err.max(-1).values.median()) <= 0.2 * scale, \
        (cos, float(err.mean()), float(err.max(-1).values.median()), scale)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (11, 23, 30)]
    toks = gpu.generate(prompts, 8).tokens
    eager = LLMEngine(MlaModel(cfg, gpu.model.w), max_batch=4, max_seq_len=128, use_graphs=False)
    assert torch.equal(eager.generate(prompts, 8).tokens, toks)
    # chunked prefill (attention over cached past keys) gives the same continuation
    parts = LLMEngine(MlaModel(cfg, gpu.model.w), max_batch=4, max_seq_len=128, prefill_chunk=16)
    assert torch.equal(parts.generate(prompts, 8).tokens[:, 0], toks[:, 0])
    check_status()


def _latent_cfg(**kw):
    import dataclasses
    base = MlaConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=4,
                     head_dim=256, rope_theta=1e4, rms_eps=1e-6, num_experts=8, top_k=2, moe_intermediate=128,
                     shared_intermediate=128, router="sigmoid", n_group=2, topk_group=1, routed_scale=2.5,
                     first_dense_layers=2, q_lora_rank=128, kv_lora_rank=512, absorbed=True, name="latent-cache-test")
    return dataclasses.replace(base, **kw) if kw else base


def test_latent_cache_kernels_match_reference():
    """The 576-wide shared-row decode attention and its cache writer against the fp32 restatement over the same pages
    (16 and 20 heads: a full and a ragged head tile; one and several KV splits; ragged sequence lengths)."""
    from mfq_b200.engine.kv_cache import PagedKVCache
    from mfq_b200.ops import mla as mla_ops
    from mfq_b200.ops import reference as ref
    require_gpu_lib()
    g = torch.Generator().manual_seed(0)
    lens = [1, 16, 77, 300]
    b, ps = len(lens), 16
    for heads, splits in ((16, 1), (20, 3)):
        cache = PagedKVCache(layers=1, kv_heads=1, head_dim=576, num_pages=128, max_seqs=b, max_pages_per_seq=24, device="cuda")
        kv = cache.layer(0)
        for r, n in enumerate(lens):
            cache.assign(r, 900 + r, n)
            rows = (torch.randn((n, 576), generator=g) * 0.7).to(torch.bfloat16).cuda()
            mla_ops.latent_write(rows, cache.slots(900 + r, 0, n).cuda(), kv)
        q = (torch.randn((b, heads, 576), generator=g) * 0.3).to(torch.bfloat16).cuda()
        seq_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
        got = mla_ops.decode(q, kv, cache.block_table[:b], seq_lens, sm_scale=0.07, splits=splits).float().cpu()
        check_status()
        # reference: the dequantized pages as one KV head, values = latent part of the same row
        want = ref.paged_attn_decode(q.cpu(), _cpu_layer(kv), cache.block_table[:b].cpu(), seq_lens.cpu(), 0.07, 1).float()[:, :, :512]
        err = (got - want).abs().max() / want.abs().max()
        assert float(err) < 2e-2, (heads, splits, float(err))


def _cpu_layer(kv):
    from mfq_b200.engine.kv_cache import LayerKV
    return LayerKV(kv.k.cpu(), kv.v.cpu(), kv.k_scale.cpu(), kv.v_scale.cpu(), kv.page_size)


def test_latent_cache_model_matches_cpu_and_decodes_under_graphs():
    """The weight-absorbed model on the GPU (latent cache, shared-row decode kernel) against its CPU restatement."""
    require_gpu_lib()
    cfg = _latent_cfg()
    w_cpu = random_mla_weights(cfg, "cpu", seed=5, std=0.05, expert_chunk=3)
    gpu = LLMEngine(MlaModel(cfg, _to(w_cpu, "cuda")), max_batch=4, max_seq_len=160)
    cpu = LLMEngine(MlaModel(cfg, w_cpu), max_batch=4, max_seq_len=160, device="cpu")
    assert gpu.cache.bytes_per_token() < 2 * 1300 * cfg.num_layers  # ~1.2 KB per token and layer, whatever the head count
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(3))
    lg, lc = _logits(gpu, prompt, "cuda"), _logits(cpu, prompt, "cpu")
    check_status()
    scale = float(lc.abs().max())
    cos = float(torch.nn.functional.cosine_similarity(lg.flatten(), lc.flatten(), dim=0))
    assert cos > 0.99 and float((lg - lc).abs().mean()) <= 0.03 * scale, (cos, float((lg - lc).abs().mean()), scale)
    # teacher-forced decode steps: the same tokens through both, so the step logits can be compared number by number
    def forced(eng, dev):
        n = prompt.numel()
        eng.cache.assign(0, 777, n + 6)
        step = StepBuffers(input_ids=prompt.to(dev, torch.int32), positions=torch.arange(n, dtype=torch.int32, device=dev),
                           slots=eng.cache.slots(777, 0, n).to(dev), cu_seqlens=[0, n])
        eng.model.forward(step, eng.cache, prefill=True)
        outs = []
        for j, tok in enumerate((5, 900, 17, 333, 64)):
            step = StepBuffers(input_ids=torch.tensor([tok], dtype=torch.int32, device=dev),
                               positions=torch.tensor([n + j], dtype=torch.int32, device=dev),
                               slots=eng.cache.slots(777, n + j, 1).to(dev), block_table=eng.cache.block_table[:1],
                               seq_lens=torch.tensor([n + j + 1], dtype=torch.int32, device=dev))
            outs.append(eng.model.forward(step, eng.cache, prefill=False).float().cpu())
        eng.cache.release(777)
        return torch.cat(outs, 0)
    dg, dc = forced(gpu, "cuda"), forced(cpu, "cpu")
    check_status()
    dcos = float(torch.nn.functional.cosine_similarity(dg.flatten(), dc.flatten(), dim=0))
    assert dcos > 0.99 and float((dg - dc).abs().mean()) <= 0.03 * float(dc.abs().max()), (dcos, float((dg - dc).abs().mean()))
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (11, 23, 30)]
    toks = gpu.generate(prompts, 8).tokens
    check_status()
    eager = LLMEngine(MlaModel(cfg, gpu.model.w), max_batch=4, max_seq_len=160, use_graphs=False)
    assert torch.equal(eager.generate(prompts, 8).tokens, toks)


def test_latent_cache_chunked_prefill_and_verify_window():
    """A prompt prefilled in chunks (later chunks attend to latents read back from the cache) and a three-token verify
    window over the latent cache, each against the CPU restatement of the same call."""
    require_gpu_lib()
    cfg = _latent_cfg()
    w_cpu = random_mla_weights(cfg, "cpu", seed=6, std=0.05, expert_chunk=3)
    gpu = LLMEngine(MlaModel(cfg, _to(w_cpu, "cuda")), max_batch=2, max_seq_len=160, prefill_chunk=16, use_graphs=False)
    whole = LLMEngine(MlaModel(cfg, gpu.model.w), max_batch=2, max_seq_len=160, use_graphs=False)
    cpu = LLMEngine(MlaModel(cfg, w_cpu), max_batch=2, max_seq_len=160, device="cpu")
    prompt = torch.randint(0, cfg.vocab_size, (45,), generator=torch.Generator().manual_seed(8))

    def chunked_logits(eng, dev, chunk):
        n = prompt.numel()
        eng.cache.assign(0, 321, n + 4)
        last = None
        for a in range(0, n, chunk):
            b = min(n, a + chunk)
            step = StepBuffers(input_ids=prompt[a:b].to(dev, torch.int32), positions=torch.arange(a, b, dtype=torch.int32, device=dev),
                               slots=eng.cache.slots(321, a, b - a).to(dev), cu_seqlens=[0, b - a], past_len=a,
                               block_table=eng.cache.block_table[:1])
            last = eng.model.forward(step, eng.cache, prefill=True).float().cpu()
        return last, n

    lc, n = chunked_logits(gpu, "cuda", 16)
    lw, _ = chunked_logits(whole, "cuda", 64)
    check_status()
    cos = float(torch.nn.functional.cosine_similarity(lc.flatten(), lw[-lc.shape[0]:].flatten(), dim=0))
    assert cos > 0.995, cos  # the past seen through its FP8 cache rows instead of the bf16 values of the same chunk
    lr, _ = chunked_logits(cpu, "cpu", 16)
    cos = float(torch.nn.functional.cosine_similarity(lc.flatten(), lr.flatten(), dim=0))
    assert cos > 0.99, cos

    # three-token window after the prompt (rows 0 of both engines still hold it)
    def window(eng, dev):
        toks = torch.tensor([7, 300, 41], dtype=torch.int32, device=dev)
        step = StepBuffers(input_ids=toks, positions=torch.arange(n, n + 3, dtype=torch.int32, device=dev),
                           slots=eng.cache.slots(321, n, 3).to(dev), block_table=eng.cache.block_table[:1],
                           seq_lens=torch.tensor([n + 3], dtype=torch.int32, device=dev), q_len=3)
        return eng.model.forward(step, eng.cache, prefill=False, gather_logits=False).float().cpu()
    wg, wc = window(gpu, "cuda"), window(cpu, "cpu")
    check_status()
    assert wg.shape == wc.shape and wg.shape[0] == 3
    cos = float(torch.nn.functional.cosine_similarity(wg.flatten(), wc.flatten(), dim=0))
    assert cos > 0.99 and float((wg - wc).abs().mean()) <= 0.03 * float(wc.abs().max()), cos

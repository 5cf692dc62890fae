"""tcgen05 prefill attention against the fp32 reference."""

import math

import pytest
import torch

from mfq_b200 import ops
from mfq_b200.ops import reference as ref
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,hq,hk", [(128, 4, 2), (300, 8, 2), (1024, 4, 4), (1, 4, 1), (129, 2, 1)])
def test_prefill_attention_matches_reference(t, hq, hk):
    require_gpu_lib()
    g = torch.Generator(device="cuda").manual_seed(t)
    q = torch.randn((t, hq, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((t, hk, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((t, hk, 128), generator=g, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(128)
    got = ops.kernels.attn_prefill_bf16(q, k, v, scale)
    check_status()
    want = ref.attention(q, k, v, scale, causal_offset=0)
    assert_close(got, want, rel=2e-2, what=f"prefill attention T={t}")


@pytest.mark.parametrize("t,past,hq,hk", [(128, 0, 4, 2), (300, 0, 8, 1), (1024, 0, 2, 2), (1, 0, 4, 1), (200, 77, 8, 2),
                                           (64, 1000, 4, 1), (2048, 0, 2, 1)])
def test_prefill_attention_head_dim_256(t, past, hq, hk):
    """The 256-wide kernel keeps O in TMEM and rescales it lazily; large-magnitude late keys force rescales."""
    require_gpu_lib()
    g = torch.Generator(device="cuda").manual_seed(7 * t + past)
    q = torch.randn((t, hq, 256), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((past + t, hk, 256), generator=g, device="cuda")
    # growing key magnitude: the running maximum keeps rising, so the rescale path runs many times
    k = (k * torch.linspace(0.5, 3.0, past + t, device="cuda")[:, None, None]).to(torch.bfloat16)
    v = torch.randn((past + t, hk, 256), generator=g, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(256)
    got = ops.kernels.attn_prefill_bf16(q, k, v, scale)
    check_status()
    want = ref.attention(q, k, v, scale, causal_offset=past)
    assert_close(got, want, rel=2e-2, what=f"prefill attention D=256 T={t} past={past}")


def test_packed_sequences_do_not_mix():
    require_gpu_lib()
    q = torch.randn((200, 4, 128), device="cuda").to(torch.bfloat16)
    k = torch.randn((200, 2, 128), device="cuda").to(torch.bfloat16)
    v = torch.randn((200, 2, 128), device="cuda").to(torch.bfloat16)
    got = ops.attn_prefill(q, k, v, [0, 70, 200], 0.09)
    want = torch.cat([ref.attention(q[:70], k[:70], v[:70], 0.09, 0), ref.attention(q[70:], k[70:], v[70:], 0.09, 0)])
    assert_close(got, want, rel=2e-2)
    check_status()


@pytest.mark.parametrize("tq,past", [(128, 128), (200, 77), (64, 1000), (300, 1)])
def test_prefill_attention_with_past_keys(tq, past):
    """Queries of a later chunk attend to the cached past + the chunk (causal with an offset)."""
    import torch
    from mfq_b200.ops import kernels as K
    from mfq_b200.ops import reference as ref
    from gpu_common import assert_close, check_status, require_gpu_lib
    require_gpu_lib()
    g = torch.Generator(device="cuda").manual_seed(tq + past)
    hq, hk, d = 8, 2, 128
    q = torch.randn((tq, hq, d), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((past + tq, hk, d), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((past + tq, hk, d), generator=g, device="cuda").to(torch.bfloat16)
    got = K.attn_prefill_bf16(q, k, v, 0.088)
    check_status()
    want = ref.attention(q, k, v, 0.088, causal_offset=past)
    assert_close(got.float(), want.float(), rel=2e-2, what="prefill attention with past")


def test_kv_gather_dequant_and_chunked_engine_prefill():
    import torch
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    from mfq_b200.ops import kernels as K
    from mfq_b200.ops import reference as ref
    from gpu_common import assert_close, check_status, require_gpu_lib
    require_gpu_lib()
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cuda", seed=2, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (300,), generator=torch.Generator().manual_seed(3))
    whole = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=512)
    parts = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=512, prefill_chunk=128)
    a = whole.generate([prompt], 8).tokens[0].tolist()
    b = parts.generate([prompt], 8).tokens[0].tolist()
    check_status()
    n = 0
    while n < 8 and a[n] == b[n]:
        n += 1
    assert n >= 6, (a, b)  # chunk boundaries change the summation order of the attention slightly
    # the gather kernel returns exactly what the pages hold
    kv = parts.cache.layer(0)
    row = parts.cache.block_table[0]
    kd, vd = K.kv_gather_dequant(kv, row, 200)
    t = torch.arange(200, device="cuda")
    kr, vr = ref.gather_slots(kv, row[(t // 16).long()] * 16 + t % 16)
    assert_close(kd.float(), kr.float(), rel=1e-2, what="gathered K")
    assert_close(vd.float(), vr.float(), rel=1e-2, what="gathered V")


def test_prefix_cache_restores_pages_on_gpu(tmp_path):
    import torch
    from mfq_b200 import native
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    from gpu_common import check_status, require_gpu_lib
    require_gpu_lib()
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cuda", seed=2, std=0.05)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, cfg.vocab_size, (300,), generator=g)
    p1 = torch.cat([shared, torch.randint(0, cfg.vocab_size, (20,), generator=g)])
    pc = native.PrefixCache(tmp_path / "kv", ram_budget=256 << 20, disk_budget=0, block_tokens=256)
    eng = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=512, prefix_cache=pc, prefix_salt="tiny")
    first = eng.generate([p1], 6).tokens[0].tolist()
    assert eng.prefix_stats["blocks_stored"] == 1
    eng.release(0)
    again = eng.generate([p1], 6).tokens[0].tolist()  # 256 tokens restored, 64 recomputed against them
    check_status()
    assert eng.prefix_stats["blocks_hit"] == 1
    n = 0
    while n < 6 and first[n] == again[n]:
        n += 1
    assert n >= 5, (first, again)
    pc.close()

"""Fused memory-bound kernels against their fp32 PyTorch restatements."""

import math

import pytest
import torch

from mfq_b200 import ops
from mfq_b200.engine.kv_cache import PagedKVCache
from mfq_b200.ops import reference as ref
from gpu_common import assert_close, require_gpu_lib

pytestmark = pytest.mark.gpu


def deq(q, s):
    return q.float() * s[:, None]


@pytest.mark.parametrize("m,h", [(1, 256), (7, 4096), (33, 2048), (4, 7168)])
def test_rmsnorm_quant(m, h):
    require_gpu_lib()
    x = torch.randn((m, h), device="cuda").to(torch.bfloat16)
    r = torch.randn((m, h), device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16)
    q, s, y, nr = ops.rmsnorm_quant(x, w, 1e-5, residual=r, want_y=True)
    q2, s2, y2, nr2 = ref.rmsnorm_quant(x, w, 1e-5, residual=r)
    assert torch.equal(nr, nr2)
    assert_close(y, y2, rel=1e-2, what="norm")
    assert_close(s, s2, rel=1e-2, what="scale")
    assert_close(deq(q, s), y2, rel=0.07, what="fp8 rows")
    q3, s3, _, _ = ops.rmsnorm_quant(x, w, 1e-5)
    assert_close(deq(q3, s3), ref.rmsnorm(x, w, 1e-5), rel=0.07, what="no residual")


def test_quant_rows_and_swiglu():
    require_gpu_lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn((9, 1024), device="cuda", generator=g).to(torch.bfloat16)
    q, s = ops.quant_rows(x)
    q2, s2 = ref.quant_rows(x)
    assert_close(s, s2, rel=1e-5, what="row scale")
    assert (q.float() - q2.float()).abs().max() <= 32, "codes may differ by at most one step"
    assert_close(deq(q, s), x, rel=0.07)  # E4M3 keeps three mantissa bits: at most 6.25 % off per element
    gu = torch.randn((9, 2 * 1536), device="cuda", generator=g).to(torch.bfloat16)
    q, s = ops.silu_mul_quant(gu)
    q2, s2 = ref.silu_mul_quant(gu)
    assert_close(s, s2, rel=1e-2)
    # the kernel rounds silu(g) * u once, the restatement goes through bf16 first: a product that lands on a rounding
    # boundary takes the neighbouring code (one step = 12.5 %), so a small share of the elements may differ by a step
    assert_close(deq(q, s), deq(q2, s2), rel=0.07, outliers=3e-2)
    # decode-sized batches of wide rows take the kernel that splits a row over a cluster of four CTAs
    for m, i in ((64, 14336), (5, 4096), (3, 5120)):
        gu = torch.randn((m, 2 * i), device="cuda", generator=g).to(torch.bfloat16)
        q, s = ops.silu_mul_quant(gu)
        q2, s2 = ref.silu_mul_quant(gu)
        assert_close(s, s2, rel=1e-2, what=f"swiglu scale {m}x{i}")
        assert_close(deq(q, s), deq(q2, s2), rel=0.07, outliers=3e-2, what=f"swiglu rows {m}x{i}")


def make_cache(hk, d, batch, max_len):
    pages = batch * math.ceil(max_len / 16) + 1
    return PagedKVCache(layers=1, kv_heads=hk, head_dim=d, num_pages=pages, max_seqs=batch,
                        max_pages_per_seq=math.ceil(max_len / 16), device="cuda")


@pytest.mark.parametrize("hq,hk,d", [(8, 2, 128), (4, 4, 128), (4, 2, 64), (16, 2, 256), (4, 1, 256)])
def test_rope_kv_write_and_decode_attention(hq, hk, d):
    require_gpu_lib()
    lens = [1, 17, 200, 513]
    b = len(lens)
    cache = make_cache(hk, d, b, 1024)
    kv = cache.layer(0)
    ref_cache = make_cache(hk, d, b, 1024)
    rkv = ref_cache.layer(0)
    theta = 1e4
    for i, n in enumerate(lens):
        cache.assign(i, i, n)
        ref_cache.assign(i, i, n)
        qkv = torch.randn((n, (hq + 2 * hk) * d), device="cuda").to(torch.bfloat16)
        pos = torch.arange(n, dtype=torch.int32, device="cuda")
        slots = cache.slots(i, 0, n).cuda()
        q = ops.rope_kv_write(qkv, pos, slots, kv, n_q=hq, n_kv=hk, head_dim=d, theta=theta)
        q3 = qkv.view(n, hq + 2 * hk, d)
        q_ref = ref.rope(q3[:, :hq], pos, theta)
        k_ref = ref.rope(q3[:, hq : hq + hk], pos, theta)
        ref.write_kv(rkv, k_ref, q3[:, hq + hk :], ref_cache.slots(i, 0, n).cuda())
        assert_close(q, q_ref, rel=1e-2, what="rope q")
    assert torch.equal(cache.block_table, ref_cache.block_table)
    from mfq_b200.engine.kv_cache import k_logical, v_logical
    k_mine = k_logical(kv.k).float() * kv.k_scale[..., None]
    k_theirs = k_logical(rkv.k).float() * rkv.k_scale[..., None]
    assert_close(k_mine, k_theirs, rel=0.07, what="k pages")
    assert_close(v_logical(kv.v).float() * kv.v_scale[..., None], v_logical(rkv.v).float() * rkv.v_scale[..., None],
                 rel=0.07, what="v pages")
    q = torch.randn((b, hq, d), device="cuda").to(torch.bfloat16)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    want = ref.paged_attn_decode(q, kv, cache.block_table, seq_lens, 1 / math.sqrt(d))
    for splits in (1, 3, 8, 40):
        got = ops.paged_attn_decode(q, kv, cache.block_table, seq_lens, sm_scale=1 / math.sqrt(d), splits=splits)
        assert_close(got, want, rel=2e-2, what=f"decode attention splits={splits}")


@pytest.mark.parametrize("hq,hk,d,ql", [(8, 2, 128, 4), (8, 2, 128, 2), (4, 4, 128, 3), (8, 1, 256, 1), (16, 2, 256, 2)])
def test_decode_attention_verify_window(hq, hk, d, ql):
    """Windows of several query tokens: 16 (row, head) pairs take the 16-row kernel, up to 8 the tokens-as-rows one."""
    require_gpu_lib()
    n = 100
    cache = make_cache(hk, d, 1, 256)
    kv = cache.layer(0)
    cache.assign(0, 0, n)
    qkv = torch.randn((n, (hq + 2 * hk) * d), device="cuda").to(torch.bfloat16)
    ops.rope_kv_write(qkv, torch.arange(n, dtype=torch.int32, device="cuda"), cache.slots(0, 0, n).cuda(), kv, n_q=hq,
                      n_kv=hk, head_dim=d, theta=1e4)
    q = torch.randn((ql, hq, d), device="cuda").to(torch.bfloat16)
    sl = torch.tensor([n], dtype=torch.int32, device="cuda")
    want = ref.paged_attn_decode(q, kv, cache.block_table, sl, 0.1, q_len=ql)
    got = ops.paged_attn_decode(q, kv, cache.block_table, sl, sm_scale=0.1, splits=2, q_len=ql)
    assert_close(got, want, rel=2e-2)


def test_argmax_embed_advance():
    require_gpu_lib()
    logits = torch.randn((5, 128256), device="cuda").to(torch.bfloat16)
    logits[2, 7] = logits[2, 100000] = 50.0
    got = ops.argmax(logits)
    assert got.tolist() == logits.float().argmax(-1).tolist() and got[2].item() == 7
    table = torch.randn((1000, 256), device="cuda").to(torch.bfloat16)
    ids = torch.tensor([3, 999, 0], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.embed(ids, table), table[ids.long()])
    bt = torch.arange(40, dtype=torch.int32, device="cuda").reshape(2, 20) + 1
    sampled = torch.tensor([11, 12], dtype=torch.int32, device="cuda")
    ids = torch.zeros(2, dtype=torch.int32, device="cuda")
    pos = torch.zeros(2, dtype=torch.int32, device="cuda")
    sl = torch.tensor([15, 16], dtype=torch.int32, device="cuda")
    slots = torch.zeros(2, dtype=torch.int32, device="cuda")
    ops.decode_advance(sampled, ids, pos, sl, slots, bt, 16)
    assert ids.tolist() == [11, 12] and pos.tolist() == [15, 16] and sl.tolist() == [16, 17]
    assert slots.tolist() == [1 * 16 + 15, 22 * 16 + 0]


def test_diagnose_kernel_checks_pass():
    require_gpu_lib()
    from mfq_b200 import diagnostics
    report = diagnostics.run()
    failed = {k: v for k, v in report["checks"].items() if not v["ok"]}
    assert report["ok"], (failed, report.get("device_status"))
    assert {"fp8-gemm", "attention", "engine", "gdn-chunked", "packed-experts", "mla-latent-cache", "moe-grouped", "codecs",
            "native"} <= set(report["checks"])

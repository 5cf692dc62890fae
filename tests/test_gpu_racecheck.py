"""Every operator with scratch memory, counters or cross-CTA hand-overs gives the same bits on every launch, with its
scratch poisoned in between (what a race or a read of stale scratch would break)."""

import math

import pytest
import torch

from mfq_b200 import ops
from mfq_b200.engine.kv_cache import PagedKVCache
from mfq_b200.ops import moe as moe_ops
from mfq_b200.ops import reference as ref
from mfq_b200.quantize.fp8_block import quantize_fp8_block_torch
from mfq_b200.utils import racecheck
from gpu_common import require_gpu_lib

pytestmark = pytest.mark.gpu


def _gemm_inputs(m, n, k, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    return (*ref.quant_rows(x), *quantize_fp8_block_torch(w), torch.randn((m, n), generator=g, device="cuda").to(torch.bfloat16))


@pytest.mark.parametrize("m,n,k,splits", [(64, 4096, 4096, 4), (64, 6144, 4096, 3), (20, 512, 4096, 16), (300, 1024, 2048, 2), (8, 4096, 4096, None)])
def test_gemm_paths_are_launch_invariant(m, n, k, splits):
    """Cluster split-K (up to 8 splits), the global-scratch path with its arrival counters (16), and the GEMV."""
    require_gpu_lib()
    xq, xs, wq, ws, res = _gemm_inputs(m, n, k)
    rep = racecheck.check(f"gemm {m}x{n}x{k} s{splits}", lambda: ops.fp8_gemm(xq, xs, wq, ws, residual=res, splits=splits))
    assert rep.ok, rep


def test_split_attention_and_its_merge_are_launch_invariant():
    require_gpu_lib()
    hq, hk, d, lens = 8, 2, 128, [5, 200, 513, 1000]
    b = len(lens)
    cache = PagedKVCache(layers=1, kv_heads=hk, head_dim=d, num_pages=b * 64 + 1, max_seqs=b, max_pages_per_seq=64, device="cuda")
    kv = cache.layer(0)
    g = torch.Generator(device="cuda").manual_seed(1)
    for i, n in enumerate(lens):
        cache.assign(i, i, n)
        qkv = torch.randn((n, (hq + 2 * hk) * d), generator=g, device="cuda").to(torch.bfloat16)
        ops.rope_kv_write(qkv, torch.arange(n, dtype=torch.int32, device="cuda"), cache.slots(i, 0, n).cuda(), kv, n_q=hq, n_kv=hk,
                          head_dim=d, theta=1e4)
    q = torch.randn((b, hq, d), generator=g, device="cuda").to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    for splits in (1, 3, 8):
        rep = racecheck.check(f"attention splits={splits}",
                              lambda: ops.paged_attn_decode(q, kv, cache.block_table, sl, sm_scale=1 / math.sqrt(d), splits=splits))
        assert rep.ok, rep


def test_moe_layer_is_launch_invariant():
    """Route plan (shared-memory counts and scans), grouped GEMMs, weighted combine."""
    require_gpu_lib()
    e, h, inter, t, k = 8, 512, 256, 40, 2
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((t, h), generator=g, device="cuda").to(torch.bfloat16)
    router = (torch.randn((e, h), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    gu = [quantize_fp8_block_torch((torch.randn((2 * inter, h), generator=g, device="cuda") * 0.05).to(torch.bfloat16)) for _ in range(e)]
    dn = [quantize_fp8_block_torch((torch.randn((h, inter), generator=g, device="cuda") * 0.05).to(torch.bfloat16)) for _ in range(e)]
    gu_q, gu_s = torch.stack([a for a, _ in gu]), torch.stack([b for _, b in gu])
    dn_q, dn_s = torch.stack([a for a, _ in dn]), torch.stack([b for _, b in dn])
    xq, xs = ref.quant_rows(x)

    def layer():
        ids, wt = moe_ops.router_topk(x, router, k)
        return ids, moe_ops.moe_ffn_fp8(xq, xs, ids, wt, gu_q, gu_s, dn_q, dn_s)
    rep = racecheck.check("moe layer", layer)
    assert rep.ok, rep


def test_the_check_itself_notices_a_dependence_on_scratch():
    """A function whose result depends on the (poisoned) scratch is reported, so a pass above means something."""
    require_gpu_lib()
    ws = ops.Workspace.get(torch.device("cuda"))
    rep = racecheck.check("reads scratch", lambda: ws.attn_acc[:16].clone())
    assert not rep.finite and not rep.ok
    calls = [0]

    def drifting():
        calls[0] += 1
        return torch.full((4,), float(calls[0]), device="cuda")
    rep = racecheck.check("order dependent", drifting)
    assert not rep.bit_identical and rep.finite

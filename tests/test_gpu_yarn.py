"""Rotary kernel with YaRN context extension against the fp32 restatement (full and partial rotary)."""

import math

import pytest
import torch

from mfq_b200 import ops
from mfq_b200.engine.kv_cache import PagedKVCache, k_logical
from mfq_b200.models.rope_scaling import YarnScaling
from mfq_b200.ops import reference as ref
from gpu_common import assert_close, require_gpu_lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,rot", [(128, None), (64, None), (256, 64)])
def test_rope_kv_write_with_yarn(d, rot):
    require_gpu_lib()
    hq, hk, n = 4, 2, 96
    y = YarnScaling(factor=4.0, original_max_position=2048)
    pages = math.ceil(n / 16) + 1
    cache = PagedKVCache(layers=1, kv_heads=hk, head_dim=d, num_pages=pages, max_seqs=1, max_pages_per_seq=pages - 1, device="cuda")
    rcache = PagedKVCache(layers=1, kv_heads=hk, head_dim=d, num_pages=pages, max_seqs=1, max_pages_per_seq=pages - 1, device="cuda")
    cache.assign(0, 0, n)
    rcache.assign(0, 0, n)
    qkv = torch.randn((n, (hq + 2 * hk) * d), device="cuda").to(torch.bfloat16)
    # positions far beyond the trained context, where plain and scaled rotations differ in every slow pair
    pos = (torch.arange(n, dtype=torch.int32, device="cuda") * 83) % 8000
    slots = cache.slots(0, 0, n).cuda()
    q = ops.rope_kv_write(qkv, pos, slots, cache.layer(0), n_q=hq, n_kv=hk, head_dim=d, theta=1e4, rot=rot, scaling=y)
    q3 = qkv.view(n, hq + 2 * hk, d)
    q_ref = ref.rope(q3[:, :hq], pos, 1e4, rot, y)
    assert_close(q, q_ref, rel=1e-2, what="yarn q")
    plain = ref.rope(q3[:, :hq], pos, 1e4, rot)
    assert (q.float() - plain.float()).abs().max() > 0.5, "the scaled rotation must differ from the plain one out here"
    k_ref = ref.rope(q3[:, hq : hq + hk], pos, 1e4, rot, y)
    ref.write_kv(rcache.layer(0), k_ref, q3[:, hq + hk :], rcache.slots(0, 0, n).cuda())
    kv, rkv = cache.layer(0), rcache.layer(0)
    assert_close(k_logical(kv.k).float() * kv.k_scale[..., None], k_logical(rkv.k).float() * rkv.k_scale[..., None], rel=0.07,
                 what="yarn k pages")
    # factor 1 through the same entry point is the plain rotation, bit for bit
    same = ops.rope_kv_write(qkv, pos, slots, cache.layer(0), n_q=hq, n_kv=hk, head_dim=d, theta=1e4, rot=rot, scaling=YarnScaling())
    base = ops.rope_kv_write(qkv, pos, slots, cache.layer(0), n_q=hq, n_kv=hk, head_dim=d, theta=1e4, rot=rot)
    assert torch.equal(same, base)

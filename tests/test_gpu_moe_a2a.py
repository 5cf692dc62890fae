"""Expert-parallel dispatch/combine kernels on one GPU (world 1: every table is local) against the unsharded MoE path."""

import pytest
import torch

from mfq_b200.ops import moe
from mfq_b200.ops import reference as ref
from mfq_b200.quantize.fp8_block import quantize_fp8_block_torch
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def _experts(n, h, inter, g):
    gu = (torch.randn((n, 2 * inter, h), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    dn = (torch.randn((n, h, inter), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    gq, gs = zip(*[quantize_fp8_block_torch(m) for m in gu])
    dq, ds = zip(*[quantize_fp8_block_torch(m) for m in dn])
    return torch.stack(gq), torch.stack(gs), torch.stack(dq), torch.stack(ds)


@pytest.mark.parametrize("t,cap,e,k", [(1, 4, 8, 2), (37, 64, 16, 4), (200, 200, 32, 8)])
def test_dispatch_combine_world1_matches_local_moe(t, cap, e, k):
    require_gpu_lib()
    from mfq_b200.parallel.expert_parallel import ExpertParallel
    h, inter = 512, 256
    g = torch.Generator(device="cuda").manual_seed(t)
    x = torch.randn((t, h), generator=g, device="cuda").to(torch.bfloat16)
    gq, gs, dq, ds = _experts(e, h, inter, g)
    ids = torch.stack([torch.randperm(e, generator=g, device="cuda")[:k] for _ in range(t)]).to(torch.int32)
    wt = torch.rand((t, k), generator=g, device="cuda")
    base = torch.randn((t, h), generator=g, device="cuda").to(torch.bfloat16)
    xq, xs = ref.quant_rows(x)
    want = moe.moe_ffn_fp8(xq, xs, ids, wt, gq, gs, dq, ds, base=base).float()
    ep = ExpertParallel(None, torch.device("cuda"), num_experts=e, top_k=k, hidden=h, max_tokens=256)
    for _ in range(3):  # repeated calls reuse the tables and the counting flags
        recv = ep.dispatch(xq, xs, ids, wt, cap)
        assert int(recv.total.item()) == t
        assert int((recv.ids[:, 0] >= 0).sum().item()) == t
        # every token arrives exactly once, with its own multiplier and routing list
        slots = recv.send_slot[:, 0].long()
        assert torch.equal(slots.sort().values, torch.arange(t, device="cuda"))
        assert torch.equal(recv.x_q[slots].view(torch.uint8), xq.view(torch.uint8))
        assert torch.equal(recv.x_scale[slots], xs) and torch.equal(recv.ids[slots], ids)
        plan = moe.plan_routes(recv.ids, 0, e)
        xq_s, xs_s = moe.gather_rows(recv.x_q, recv.x_scale, plan)
        gu = moe.fp8_gemm_grouped(xq_s, xs_s, gq, gs, plan)
        from mfq_b200.ops import kernels as K
        hq, hs = K.silu_mul_quant(gu)
        y = moe.fp8_gemm_grouped(hq, hs, dq, ds, plan)
        got = ep.combine(y, plan, recv, base=base)
        check_status()
        # the a2a path rounds the weighted expert sum to bf16 before adding the residual
        assert_close(got.float(), want, rel=1.5e-2, what="a2a moe")
    got2 = ep.moe_ffn(xq, xs, ids, wt, gq, gs, dq, ds, base=base, cap=cap)
    check_status()
    assert torch.equal(got2, got)

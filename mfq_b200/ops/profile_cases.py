"""Small, self-terminating kernel cases for profiler captures: ``python -m mfq_b200.ops.profile_cases <case>``.

Each case launches one kernel three times on inputs of a few hundred MB (larger than the 126 MB L2, small enough
for a multi-pass capture to finish in about a minute) and exits.  Cases: ``gemm_prefill`` (M=4096, N=K=4096),
``gemm_decode`` (M=64, N=28672, K=4096), ``attn_decode`` (64 sequences x 4096 tokens), ``attn_prefill`` (T=2048),
``w4_decode`` / ``w4_prefill`` (the 4-bit in-pipeline-decode GEMM at the same shapes), ``gdn_decode`` (Gated DeltaNet step,
64 sequences), ``moe_dispatch`` (expert-parallel dispatch + combine kernels at world 1, 4096 tokens), ``gemv_decode``
(the weight-streaming FP8 kernel, M=1, N=28672, K=4096), ``attn_prefill_d256`` (T=2048, 16 query / 2 KV heads of 256),
``gdn_prefill`` (the long-row Gated DeltaNet path, 2048 tokens, 32 heads), ``mla_decode`` (latent-cache decode attention), ``packed_decode`` / ``packed_decode_bs1`` (the
packed-expert product at 64 tokens / one token, 512 experts).
"""

from __future__ import annotations

import math
import sys

import torch

from . import kernels as K
from ..engine.kv_cache import PagedKVCache


def _fp8(shape):
    return torch.randint(-100, 100, shape, device="cuda", dtype=torch.int8).view(torch.float8_e4m3fn)


def gemm(m: int, n: int, k: int) -> None:
    w = [_fp8((n, k)) for _ in range(3)]
    ws = torch.rand((math.ceil(n / 128), k // 128), device="cuda") * 0.01 + 0.001
    x, xs = _fp8((m, k)), torch.rand(m, device="cuda") * 0.01
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    for i in range(3):
        K.fp8_gemm(x, xs, w[i], ws, out=out)


def attn_decode() -> None:
    batch, ctx, hq, hk, d = 64, 4096, 32, 8, 128
    pages = math.ceil(ctx / 16)
    cache = PagedKVCache(layers=3, kv_heads=hk, head_dim=d, num_pages=batch * pages + 1, max_seqs=batch,
                         max_pages_per_seq=pages, device="cuda")
    cache.k.view(torch.int8).random_(-100, 100)
    cache.v.view(torch.int8).random_(-100, 100)
    cache.k_scale.fill_(0.01)
    cache.v_scale.fill_(0.01)
    for b in range(batch):
        cache.assign(b, b, ctx)
    q = torch.randn((batch, hq, d), device="cuda").to(torch.bfloat16)
    sl = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    for i in range(3):
        K.paged_attn_decode(q, cache.layer(i), cache.block_table, sl, sm_scale=0.088, splits=1)


def attn_prefill() -> None:
    t, hq, hk, d = 2048, 32, 8, 128
    q = torch.randn((t, hq, d), device="cuda").to(torch.bfloat16)
    k = torch.randn((t, hk, d), device="cuda").to(torch.bfloat16)
    v = torch.randn((t, hk, d), device="cuda").to(torch.bfloat16)
    for _ in range(3):
        K.attn_prefill_bf16(q, k, v, 0.088)


def attn_prefill_d256() -> None:
    t, hq, hk, d = 2048, 16, 2, 256
    q = torch.randn((t, hq, d), device="cuda").to(torch.bfloat16)
    k = torch.randn((t, hk, d), device="cuda").to(torch.bfloat16)
    v = torch.randn((t, hk, d), device="cuda").to(torch.bfloat16)
    for _ in range(3):
        K.attn_prefill_bf16(q, k, v, 1 / 16)


def gdn_prefill() -> None:
    from . import gdn
    L, hk, hv, d = 2048, 16, 32, 128
    c = 2 * hk * d + hv * d
    x = (torch.randn((L, c), device="cuda") * 0.8).to(torch.bfloat16)
    z = torch.randn((L, hv * d), device="cuda").to(torch.bfloat16)
    a = torch.randn((L, hv), device="cuda").to(torch.bfloat16)
    b = torch.randn((L, hv), device="cuda").to(torch.bfloat16)
    w = torch.randn((c, 4), device="cuda") * 0.5
    A_log, dt_bias, norm_w = torch.randn(hv, device="cuda") * 0.5, torch.randn(hv, device="cuda") * 0.5, torch.ones(d, device="cuda")
    conv_state = torch.zeros((1, 3, c), device="cuda")
    state = torch.zeros((1, hv, d, d), device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):
        qkv = gdn.conv(x, conv_state, w, slot, L)
        gdn.recurrent(qkv, z, a, b, A_log, dt_bias, norm_w, state, slot, L, hk, hv)


def mla_decode() -> None:
    """Shared-row latent attention, 64 sequences x 4096 tokens, 16 heads (one rank's share of 128): 285 MB of rows."""
    import math

    from ..engine.kv_cache import PagedKVCache
    from . import mla as mla_ops
    batch, ctx, heads = 64, 4096, 16
    pages_per = math.ceil(ctx / 16)
    cache = PagedKVCache(layers=2, kv_heads=1, head_dim=576, num_pages=batch * pages_per + 1, max_seqs=batch,
                         max_pages_per_seq=pages_per, device="cuda")
    cache.k.view(torch.int8).random_(-100, 100)
    cache.v.view(torch.int8).random_(-100, 100)
    cache.k_scale.fill_(0.01)
    cache.v_scale.fill_(0.01)
    for b in range(batch):
        cache.assign(b, b, ctx)
    q = torch.randn((batch, heads, 576), device="cuda").to(torch.bfloat16)
    sl = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    for i in range(3):
        mla_ops.decode(q, cache.layer(i % 2), cache.block_table, sl, sm_scale=0.07, splits=2)


def w4_gemm(m: int, n: int, k: int) -> None:
    from . import w4
    base = w4.quantize_torch(torch.randn((n, k), device="cuda") * 0.02)
    ws = [base] + [w4.W4Weight(base.packed.clone(), base.group.clone(), n, k, base.group_size) for _ in range(2)]
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    for i in range(3):
        w4.w4_gemm(x, ws[i], out=out)


def gdn_decode() -> None:
    """Gated DeltaNet decode step: 64 sequences x 32 value heads, one token each (state 2 MB per sequence)."""
    from . import gdn
    b, hk, hv, d = 64, 16, 32, 128
    c = (2 * hk + hv) * d
    x = torch.randn((b, c), device="cuda").to(torch.bfloat16)
    z = torch.randn((b, hv * d), device="cuda").to(torch.bfloat16)
    a = torch.randn((b, hv), device="cuda").to(torch.bfloat16)
    bb = torch.randn((b, hv), device="cuda").to(torch.bfloat16)
    w = torch.randn((c, 4), device="cuda") * 0.5
    slot = torch.arange(b, dtype=torch.int32, device="cuda")
    states = [torch.randn((b, hv, d, d), device="cuda") * 0.1 for _ in range(3)]  # 3 x 134 MB: each launch streams its own
    conv = torch.zeros((b, 3, c), device="cuda")
    al, dt, nw = torch.zeros(hv, device="cuda"), torch.zeros(hv, device="cuda"), torch.ones(d, device="cuda")
    for i in range(3):
        qkv = gdn.conv(x, conv, w, slot, 1)
        gdn.recurrent(qkv, z, a, bb, al, dt, nw, states[i], slot, 1, hk, hv)


def moe_dispatch() -> None:
    """Dispatch + combine kernels on one GPU (world 1): 4096 tokens, hidden 7168, 256 experts, top-8."""
    from . import moe
    from ..parallel.expert_parallel import ExpertParallel
    t, h, e, k = 4096, 7168, 256, 8
    ep = ExpertParallel(None, torch.device("cuda"), num_experts=e, top_k=k, hidden=h, max_tokens=t)
    xq = _fp8((t, h))
    xs = torch.rand(t, device="cuda")
    ids = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(t)]).to(torch.int32)
    wt = torch.rand((t, k), device="cuda")
    y = torch.zeros((t * k, h), dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        recv = ep.dispatch(xq, xs, ids, wt)
        plan = moe.plan_routes(recv.ids, 0, e)
        ep.combine(y, plan, recv)


def packed_decode(tokens: int = 64) -> None:
    """Packed expert gate/up product of the 512-expert hybrid model: `tokens` tokens x top-10 routes over synthetic NINT 2-5
    bit / MXFP4 payloads ([1024, 2048] per expert, about 0.5 GB in all)."""
    from . import moe, packed
    e, k = 512, 10
    rng = torch.Generator().manual_seed(0)
    bits = [int(b) for b in torch.tensor([2, 3, 4, 5, 16])[torch.randint(0, 5, (e,), generator=rng)]]
    pe = packed.PackedExperts.synthetic(e, 1024, 2048, bits, "cuda", gs=32, seed=1)
    x = torch.randn((tokens, 2048), device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(tokens)]).to(torch.int32)
    plan = moe.plan_routes(ids, 0, e, token_tile=16)
    for _ in range(3):
        packed.packed_gemv_grouped(pe, x, plan, gather=True)


CASES = {"gemm_prefill": lambda: gemm(4096, 4096, 4096), "gemm_decode": lambda: gemm(64, 28672, 4096),
         "gemm_decode_splitk": lambda: gemm(64, 4096, 14336),
         "attn_decode": attn_decode, "attn_prefill": attn_prefill, "w4_decode": lambda: w4_gemm(64, 28672, 4096),
         "w4_prefill": lambda: w4_gemm(4096, 4096, 4096), "gdn_decode": gdn_decode, "moe_dispatch": moe_dispatch,
         "gemv_decode": lambda: gemm(1, 28672, 4096), "packed_decode": packed_decode, "packed_decode_bs1": lambda: packed_decode(1), "attn_prefill_d256": attn_prefill_d256, "gdn_prefill": gdn_prefill, "mla_decode": mla_decode}

if __name__ == "__main__":
    CASES[sys.argv[1]]()
    torch.cuda.synchronize()
    K.Workspace.get(torch.device("cuda", 0)).check()
    print("ok", sys.argv[1])

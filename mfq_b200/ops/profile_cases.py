"""Small, self-terminating kernel cases for profiler captures: ``python -m mfq_b200.ops.profile_cases <case>``.

Each case launches one kernel three times on inputs of a few hundred MB (larger than the 126 MB L2, small enough
for a multi-pass capture to finish in about a minute) and exits.  Cases: ``gemm_prefill`` (M=4096, N=K=4096),
``gemm_decode`` (M=64, N=28672, K=4096), ``attn_decode`` (64 sequences x 4096 tokens), ``attn_prefill`` (T=2048).
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


CASES = {"gemm_prefill": lambda: gemm(4096, 4096, 4096), "gemm_decode": lambda: gemm(64, 28672, 4096),
         "attn_decode": attn_decode, "attn_prefill": attn_prefill}

if __name__ == "__main__":
    CASES[sys.argv[1]]()
    torch.cuda.synchronize()
    K.Workspace.get(torch.device("cuda", 0)).check()
    print("ok", sys.argv[1])

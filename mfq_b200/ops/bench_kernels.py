"""Per-kernel timings at the Llama-8B shapes: ``python -m mfq_b200.ops.bench_kernels [--json out.json]``.

Each kernel is timed in isolation with CUDA events over ``reps`` launches after a warm-up, rotating through
enough independent weight copies that every launch reads its weights from HBM (more than 4x the 126 MB L2),
and reported against the measured roofline denominators (copy bandwidth / cuBLAS bf16 rate) when
``MEASURED_PEAKS.json`` is present in the working directory.
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import kernels as K
from . import reference as ref
from ..engine.kv_cache import PagedKVCache

L2_BYTES = 126 << 20


def time_ms(fn, reps: int, warmup: int = 3) -> float:
    """Device time per launch: ``reps`` launches captured in one CUDA graph, best of three replays (graph
    replay removes the host launch cost, which would otherwise hide kernels of a few microseconds)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn(0)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        for i in range(reps):
            fn(i)
    best = float("inf")
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / reps)
    return best


def peaks() -> dict:
    if os.path.exists("MEASURED_PEAKS.json"):
        p = json.load(open("MEASURED_PEAKS.json"))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "kind": "fallback"}


def bench_gemm(m: int, n: int, k: int, reps: int, splits=None, tile=None) -> dict:
    copies = max(1, min(16, math.ceil(4 * L2_BYTES / (n * k))))
    w = [torch.randint(-100, 100, (n, k), device="cuda", dtype=torch.int8).view(torch.float8_e4m3fn) for _ in range(copies)]
    ws = torch.rand((math.ceil(n / 128), k // 128), device="cuda") * 0.01 + 0.001
    x = torch.randint(-100, 100, (m, k), device="cuda", dtype=torch.int8).view(torch.float8_e4m3fn)
    xs = torch.rand(m, device="cuda") * 0.01 + 0.001
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    ms = time_ms(lambda i: K.fp8_gemm(x, xs, w[i % copies], ws, out=out, splits=splits, token_tile=tile), reps)
    byt = n * k + m * k + 2 * m * n
    gemv = splits is None and tile is None and K.use_gemv(m, n, k)
    return {"kernel": "fp8_gemv" if gemv else "fp8_gemm", "m": m, "n": n, "k": k, "us": ms * 1e3, "gbs": byt / ms / 1e6,
            "tflops": 2 * m * n * k / ms / 1e9, "splits": splits if splits else K.pick_splits(m, n, k)}


def bench_w4_gemm(m: int, n: int, k: int, reps: int, splits=None) -> dict:
    """4-bit in-pipeline-decode GEMM: same shapes as the FP8 GEMM, 5 bits per weight of HBM traffic."""
    from . import w4
    copies = max(1, min(16, math.ceil(4 * L2_BYTES / (n * k * 5 // 8))))
    base = w4.quantize_torch(torch.randn((n, k), device="cuda") * 0.02)
    ws = [base] + [w4.W4Weight(base.packed.clone(), base.group.clone(), n, k, base.group_size) for _ in range(copies - 1)]
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    ms = time_ms(lambda i: w4.w4_gemm(x, ws[i % copies], out=out, splits=splits), reps)
    byt = n * k * 5 // 8 + 2 * m * k + 2 * m * n
    return {"kernel": "w4_gemm", "m": m, "n": n, "k": k, "us": ms * 1e3, "gbs": byt / ms / 1e6, "tflops": 2 * m * n * k / ms / 1e9}


def bench_attn(batch: int, ctx: int, hq: int, hk: int, d: int, splits: int, reps: int) -> dict:
    pages_per = math.ceil(ctx / 16)
    layers = max(1, math.ceil(4 * L2_BYTES / (batch * ctx * hk * d * 2)))
    cache = PagedKVCache(layers=layers, kv_heads=hk, head_dim=d, num_pages=batch * pages_per + 1, max_seqs=batch,
                         max_pages_per_seq=pages_per, device="cuda")
    cache.k.view(torch.int8).random_(-100, 100)
    cache.v.view(torch.int8).random_(-100, 100)
    cache.k_scale.fill_(0.01)
    cache.v_scale.fill_(0.01)
    for b in range(batch):
        cache.assign(b, b, ctx)
    q = torch.randn((batch, hq, d), device="cuda").to(torch.bfloat16)
    sl = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    kvs = [cache.layer(i) for i in range(layers)]
    ms = time_ms(lambda i: K.paged_attn_decode(q, kvs[i % layers], cache.block_table, sl, sm_scale=0.088, splits=splits, out=out), reps)
    byt = batch * ctx * hk * (2 * d + 8)
    return {"kernel": "paged_attn_decode", "batch": batch, "ctx": ctx, "hq": hq, "hk": hk, "d": d, "splits": splits, "us": ms * 1e3, "gbs": byt / ms / 1e6}


def bench_mla_decode(batch: int, ctx: int, heads: int, splits: int, reps: int) -> dict:
    """Shared-row latent attention: 576-wide key rows and their 512-wide latent as values, one row per token."""
    from . import mla as mla_ops
    pages_per = math.ceil(ctx / 16)
    layers = max(1, math.ceil(4 * L2_BYTES / (batch * ctx * 2 * 576)))
    cache = PagedKVCache(layers=layers, kv_heads=1, head_dim=576, num_pages=batch * pages_per + 1, max_seqs=batch,
                         max_pages_per_seq=pages_per, device="cuda")
    cache.k.view(torch.int8).random_(-100, 100)
    cache.v.view(torch.int8).random_(-100, 100)
    cache.k_scale.fill_(0.01)
    cache.v_scale.fill_(0.01)
    for b in range(batch):
        cache.assign(b, b, ctx)
    q = torch.randn((batch, heads, 576), device="cuda").to(torch.bfloat16)
    sl = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    out = torch.empty((batch, heads, 512), dtype=torch.bfloat16, device="cuda")
    kvs = [cache.layer(i) for i in range(layers)]
    ms = time_ms(lambda i: mla_ops.decode(q, kvs[i % layers], cache.block_table, sl, sm_scale=0.07, splits=splits, out=out), reps)
    byt = batch * ctx * (576 + 512 + 8) * math.ceil(heads / 16)  # every 16-head tile streams the rows once
    return {"kernel": "mla_decode", "batch": batch, "ctx": ctx, "heads": heads, "splits": splits, "us": ms * 1e3,
            "gbs": byt / ms / 1e6, "unique_gbs": batch * ctx * (576 + 512 + 8) / ms / 1e6}


def bench_prefill(t: int, hq: int, hk: int, reps: int, d: int = 128) -> list[dict]:
    q = torch.randn((t, hq, d), device="cuda").to(torch.bfloat16)
    k = torch.randn((t, hk, d), device="cuda").to(torch.bfloat16)
    v = torch.randn((t, hk, d), device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    ms = time_ms(lambda _: K.attn_prefill_bf16(q, k, v, 0.088, out=out), reps)
    rows = [{"kernel": "attn_prefill_bf16", "t": t, "hq": hq, "hk": hk, "d": d, "us": ms * 1e3,
             "tflops": 4 * t * t * hq * d / 2 / ms / 1e9}]
    pages = math.ceil(t / 16)
    cache = PagedKVCache(layers=1, kv_heads=hk, head_dim=d, num_pages=pages + 1, max_seqs=1, max_pages_per_seq=pages, device="cuda")
    cache.assign(0, 0, t)
    qkv = torch.randn((t, (hq + 2 * hk) * d), device="cuda").to(torch.bfloat16)
    pos = torch.arange(t, dtype=torch.int32, device="cuda")
    slots = cache.slots(0, 0, t).cuda()
    kd, vd = torch.empty_like(k), torch.empty_like(v)
    ms = time_ms(lambda _: K.rope_kv_write(qkv, pos, slots, cache.layer(0), n_q=hq, n_kv=hk, head_dim=d, theta=5e5, q_out=out,
                                           kd_out=kd, vd_out=vd), reps)
    rows.append({"kernel": "rope_kv_write", "t": t, "us": ms * 1e3, "gbs": t * (hq + 2 * hk) * d * 5 / ms / 1e6})
    return rows


def bench_small(m: int, h: int, i: int, reps: int) -> list[dict]:
    x = torch.randn((m, h), device="cuda").to(torch.bfloat16)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    gu = torch.randn((m, 2 * i), device="cuda").to(torch.bfloat16)
    out = []
    ms = time_ms(lambda _: K.rmsnorm_quant(x, w, 1e-5), reps)
    out.append({"kernel": "rmsnorm_quant", "m": m, "h": h, "us": ms * 1e3, "gbs": m * h * 3 / ms / 1e6})
    ms = time_ms(lambda _: K.quant_rows(x), reps)
    out.append({"kernel": "quant_rows", "m": m, "h": h, "us": ms * 1e3, "gbs": m * h * 3 / ms / 1e6})
    ms = time_ms(lambda _: K.silu_mul_quant(gu), reps)
    out.append({"kernel": "silu_mul_quant", "m": m, "i": i, "us": ms * 1e3, "gbs": m * i * 5 / ms / 1e6})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default="", help="comma separated kernel families: gemm,w4,attn,mla,small,prefill")
    ap.add_argument("--tp", type=int, default=1, help="time one rank's shard of a tensor-parallel group of this size")
    args = ap.parse_args()
    pk = peaks()
    rows = []
    only = set(filter(None, args.only.split(",")))
    want = lambda family: not only or family in only
    tp = args.tp
    shapes = [("qkv", 6144 // tp, 4096), ("o_proj", 4096, 4096 // tp), ("gate_up", 28672 // tp, 4096), ("down", 4096, 14336 // tp),
              ("lm_head", 128256 // tp, 4096)]
    for m in ((1, 64) if args.quick else (1, 16, 64, 512, 4096)) if want("gemm") else ():
        for name, n, k in shapes:
            if name == "lm_head" and m > 64:
                continue
            r = bench_gemm(m, n, k, args.reps)
            r["name"] = name
            rows.append(r)
            if r["kernel"] == "fp8_gemv":  # the tcgen05 GEMM on the same shape, for comparison
                r = bench_gemm(m, n, k, args.reps, splits=K.pick_splits(m, n, k), tile=K._token_tile(m))
                r["name"] = name
                rows.append(r)
    for m in ((1, 64) if args.quick else (1, 16, 64, 512, 4096)) if want("w4") else ():
        for name, n, k in shapes[:4]:
            r = bench_w4_gemm(m, n, k, args.reps)
            r["name"] = name
            rows.append(r)
    for batch, ctx in ((1, 4096), (64, 4096)) if want("attn") else ():
        for splits in sorted({1, 4, K.attn_splits_for(batch, max(1, 8 // tp), ctx)}):
            rows.append(bench_attn(batch, ctx, 32 // tp, max(1, 8 // tp), 128, splits, args.reps))
        # 256-wide heads of the hybrid model: 16 query heads on 2 KV heads
        rows.append(bench_attn(batch, ctx, 16, 2, 256, K.attn_splits_for(batch, 2, ctx), args.reps))
    for batch, ctx in ((1, 4096), (64, 4096)) if want("mla") else ():
        for splits in ((1, 8, 16) if batch == 1 else (1, 2, 4)):
            rows.append(bench_mla_decode(batch, ctx, max(16, 128 // tp), splits, args.reps))
    for m in (1, 64, 4096) if want("small") else ():
        rows += bench_small(m, 4096, 14336, args.reps)
    for t in (1024, 4096) if want("prefill") else ():
        rows += bench_prefill(t, 32, 8, args.reps)
        rows += bench_prefill(t, 16, 2, args.reps, d=256)[:1]
    for r in rows:
        if "gbs" in r:
            r["hbm_frac"] = r["gbs"] / pk["hbm_gbs"]
        if "tflops" in r:
            r["tensor_frac_of_bf16"] = r["tflops"] / pk["tflops"]
        print(json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}))
    if args.json:
        json.dump({"peaks": pk, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()

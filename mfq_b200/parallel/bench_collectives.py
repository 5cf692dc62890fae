"""Sweep of the fused compute+collective kernels against their library (unfused GEMM + NCCL) baselines.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m mfq_b200.parallel.bench_collectives

Per case it prints one JSON line: fused and baseline time (CUDA events around one CUDA-graph replay of the op, max
over ranks of the per-rank median, L2 flushed and ranks aligned by a device-side barrier before every timed replay;
the library all-to-all baseline synchronises with the host for its split sizes and runs eagerly), the roofline time -- the slower of
FLOPs / GEMM peak and NVLink bytes / link bandwidth -- and the achieved fraction of it.

Cases: row-parallel GEMM + all-reduce (small M) / reduce-scatter (M a multiple of W*128), all-gather + column-parallel
GEMM, and MoE dispatch + combine (256 experts, top-8, hidden 7168, uniform and Zipf(1.2) expert popularity).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from ..models.llama import Fp8Linear
from ..ops import kernels as K
from ..ops import reference as ref
from ..ops.lib import Workspace
from .expert_parallel import ExpertParallel, NcclExpertParallel
from .tensor_parallel import TensorParallel

LINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU
FP8_PEAK_TFLOPS = 2 * 1590.0  # twice the measured cuBLAS bf16 burst figure


def _graphed(fn):
    """``fn`` as a CUDA-graph replay (host launch cost out of the measurement); eager if it cannot be captured."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(g):
            fn()
    except Exception:  # e.g. a library op that synchronises with the host
        torch.cuda.synchronize()
        return fn
    return g.replay


def _time(fn, tp: TensorParallel, flush: torch.Tensor, iters: int, warmup: int = 3, graph: bool = True) -> float:
    if graph:
        fn = _graphed(fn)
    pairs = []
    for i in range(warmup + iters):  # no host synchronisation inside: the host runs ahead while the flush executes
        flush.zero_()
        tp.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in pairs[warmup:]]
    t = torch.tensor([statistics.median(times)], device=flush.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _lin(n: int, k: int, dev, seed: int) -> Fp8Linear:
    g = torch.Generator(device=dev).manual_seed(seed)
    return Fp8Linear.from_float((torch.randn((n, k), generator=g, device=dev) * 0.02))


def _acts(m: int, k: int, dev, seed: int):
    g = torch.Generator(device=dev).manual_seed(seed)
    return ref.quant_rows(torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16))


def gemm_cases(tp: TensorParallel, dev, flush, args, emit) -> None:
    w, rank = tp.world, tp.rank
    kfull, n = 7168, 7168
    for m in args.m:
        # row-parallel: K sharded, partial sums reduced
        lin = _lin(n, kfull // w, dev, 1 + rank)
        xq, xs = _acts(m, kfull // w, dev, 100 + rank)
        h = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
        flops = 2.0 * m * n * kfull / w
        if m % (w * 128) == 0:
            fused = _time(lambda: tp.gemm_reduce_scatter(lin, xq, xs), tp, flush, args.iters)
            out = torch.empty((m // w, n), dtype=torch.bfloat16, device=dev)

            def base():
                partial = K.fp8_gemm(xq, xs, lin.q, lin.scale)
                dist.reduce_scatter_tensor(out, partial)
            link_bytes = (w - 1) / w * m * n * 4  # fp32 partial tiles pushed to their owners
            name = "gemm_reduce_scatter"
        else:
            fused = _time(lambda: tp.row_parallel_linear(lin, xq, xs, h), tp, flush, args.iters)

            def base():
                partial = K.fp8_gemm(xq, xs, lin.q, lin.scale)
                dist.all_reduce(partial)
                h.add_(partial)
            link_bytes = (w - 1) * m * n * 4  # one-shot: every rank reads every peer's partial
            name = "gemm_allreduce"
        baseline = _time(base, tp, flush, args.iters)
        local = _time(lambda: K.fp8_gemm(xq, xs, lin.q, lin.scale), tp, flush, args.iters)
        roof = max(flops / (FP8_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6
        emit(dict(case=name, M=m, N=n, K=kfull, fused_us=fused, nccl_us=baseline, local_gemm_us=local, roofline_us=roof,
                  frac_of_roofline=roof / fused, speedup_vs_nccl=baseline / fused))
        # column-parallel over token-sharded input: all-gather -> GEMM
        if m % w == 0 and (m // w) * kfull % 16 == 0:
            n_local = 4096
            lin2 = _lin(n_local, kfull, dev, 7 + rank)
            xq_s, xs_s = _acts(m // w, kfull, dev, 200 + rank)
            bt = K._token_tile(m)
            fused = _time(lambda: tp.allgather_gemm(lin2, xq_s, xs_s, token_tile=bt), tp, flush, args.iters)
            full_q = torch.empty((m, kfull), dtype=torch.uint8, device=dev)
            full_s = torch.empty((m,), dtype=torch.float32, device=dev)

            def base2():
                dist.all_gather_into_tensor(full_q, xq_s.view(torch.uint8))
                dist.all_gather_into_tensor(full_s, xs_s)
                K.fp8_gemm(full_q.view(torch.float8_e4m3fn), full_s, lin2.q, lin2.scale)
            baseline = _time(base2, tp, flush, args.iters)
            flops = 2.0 * m * n_local * kfull
            link_bytes = (w - 1) / w * m * (kfull + 4)
            roof = max(flops / (FP8_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6
            emit(dict(case="allgather_gemm", M=m, N=n_local, K=kfull, fused_us=fused, nccl_us=baseline, roofline_us=roof,
                      frac_of_roofline=roof / fused, speedup_vs_nccl=baseline / fused))


def a2a_cases(tp: TensorParallel, dev, flush, args, emit) -> None:
    w, rank = tp.world, tp.rank
    hidden, experts, topk = 7168, 256, 8
    cap_max = max(1, max(args.tokens) // w)
    ep = ExpertParallel(dist.group.WORLD, dev, num_experts=experts, top_k=topk, hidden=hidden, max_tokens=cap_max)
    nep = NcclExpertParallel(dist.group.WORLD, dev, num_experts=experts, top_k=topk, hidden=hidden, max_tokens=0)
    from ..ops import moe as moe_ops
    for dist_name in ("uniform", "zipf1.2"):
        prob = torch.ones(experts) if dist_name == "uniform" else 1.0 / torch.arange(1, experts + 1).float() ** 1.2
        prob = prob[torch.randperm(experts, generator=torch.Generator().manual_seed(5))]  # hot experts spread over ranks
        for total in args.tokens:
            t = max(1, total // w)
            g = torch.Generator().manual_seed(1000 * rank + total)
            ids = torch.multinomial(prob.expand(t, experts), topk, generator=g).to(torch.int32).to(dev)
            wt = torch.rand((t, topk), generator=g).to(dev)
            xq, xs = _acts(t, hidden, dev, 300 + rank)
            e_lo = rank * ep.e_per
            state = {}

            def fused_dispatch():
                state["recv"] = ep.dispatch(xq, xs, ids, wt, cap=t)
            # the expert outputs do not matter for the timing: one zero row per routed pair
            def fused_combine():
                ep.combine(state["y"], state["plan"], state["recv"])
            evs = []
            state["y"] = torch.zeros((w * t * topk, hidden), dtype=torch.bfloat16, device=dev)

            def dispatch_and_plan():
                fused_dispatch()
                state["plan"] = moe_ops.plan_routes(state["recv"].ids, e_lo, e_lo + ep.e_per)
            # dispatch and combine must alternate strictly, also while warming up and capturing
            for _ in range(2):
                dispatch_and_plan(); fused_combine()
            torch.cuda.synchronize()
            g_d, g_c = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_d):
                dispatch_and_plan()
            with torch.cuda.graph(g_c):
                fused_combine()
            for i in range(3 + args.iters):
                flush.zero_(); tp.barrier()
                a, b, c, d = (torch.cuda.Event(enable_timing=True) for _ in range(4))
                a.record(); g_d.replay(); b.record()
                flush.zero_(); tp.barrier()
                c.record(); g_c.replay(); d.record()
                evs.append((a, b, c, d))
            torch.cuda.synchronize()
            d_times = [a.elapsed_time(b) * 1e3 for a, b, _, _ in evs[3:]]
            c_times = [c.elapsed_time(d) * 1e3 for _, _, c, d in evs[3:]]
            # library baseline
            nd, nc = [], []
            for i in range(3 + args.iters):
                flush.zero_(); tp.barrier()
                a, b, c, d = (torch.cuda.Event(enable_timing=True) for _ in range(4))
                a.record(); rx, rs_, rids, rw, ctx = nep.dispatch(xq, xs, ids, wt); b.record()
                y_tok = torch.zeros((rx.shape[0], hidden), dtype=torch.bfloat16, device=dev)
                flush.zero_(); tp.barrier()
                c.record(); nep.combine(y_tok, ctx); d.record(); d.synchronize()
                if i >= 3:
                    nd.append(a.elapsed_time(b) * 1e3); nc.append(c.elapsed_time(d) * 1e3)
            owner = torch.div(ids, ep.e_per, rounding_mode="floor")
            goes = torch.zeros((t, w), dtype=torch.bool, device=dev).scatter_(1, owner.long(), True)
            goes[:, rank] = False
            remote_rows = float(goes.sum())
            vals = torch.tensor([statistics.median(d_times), statistics.median(c_times), statistics.median(nd),
                                 statistics.median(nc), remote_rows], device=dev)
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            d_us, c_us, nd_us, nc_us, rows = (float(v) for v in vals)
            roof_d = rows * (hidden + 4 + topk * 8) / (LINK_GBS * 1e9) * 1e6
            roof_c = rows * hidden * 2 / (LINK_GBS * 1e9) * 1e6
            emit(dict(case="moe_dispatch_combine", routing=dist_name, tokens=total, tokens_per_rank=t, hidden=hidden,
                      experts=experts, top_k=topk, dispatch_us=d_us, combine_us=c_us, nccl_dispatch_us=nd_us,
                      nccl_combine_us=nc_us, roofline_dispatch_us=roof_d, roofline_combine_us=roof_c,
                      frac_of_roofline_dispatch=roof_d / d_us, frac_of_roofline_combine=roof_c / c_us,
                      speedup_vs_nccl=(nd_us + nc_us) / (d_us + c_us)))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", dest="m", type=int, nargs="*", default=[1, 16, 64, 512, 4096, 16384])
    ap.add_argument("--tokens", type=int, nargs="*", default=[1, 8, 64, 512, 2048, 8192])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip", default="", help="comma list of: gemm, a2a")
    args = ap.parse_args()
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    tp = TensorParallel(dist.group.WORLD, dev, max_rows=max(args.m + [8192]))
    flush = torch.empty(1 << 30, dtype=torch.uint8, device=dev)  # written before every timed replay: L2 flush + host slack

    def emit(rec):
        rec["world"] = tp.world
        if rank == 0:
            print("SWEEP " + json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in rec.items()}), flush=True)

    # what the method itself costs: the same flush / barrier / graph replay around a one-element kernel
    one = torch.zeros(1, device=dev)
    emit(dict(case="timing_floor", floor_us=_time(lambda: one.add_(1.0), tp, flush, args.iters)))
    if "gemm" not in args.skip:
        gemm_cases(tp, dev, flush, args, emit)
    if "a2a" not in args.skip:
        a2a_cases(tp, dev, flush, args, emit)
    torch.cuda.synchronize()
    Workspace.get(dev).check()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Mixture-of-experts operators: router top-k, route plan, grouped FP8 expert GEMMs, weighted un-permute.

``moe_ffn_fp8`` strings them together for one layer: tokens are sorted by expert (only experts in
``[e_lo, e_hi)`` -- this rank's share under expert parallelism -- get rows), one grouped GEMM computes gate/up for
all experts, SwiGLU + FP8 re-quantization runs on the sorted rows, a second grouped GEMM applies the down
projections, and the combine adds ``sum_k w[t,k] * y`` (plus the shared expert's output) to the residual.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import torch

from . import kernels as K
from .lib import Workspace, check, lib, ptr, stream_ptr

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_SIGS = {
    "mfq_moe_router_topk": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp],
    "mfq_moe_plan": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp],
    "mfq_moe_gather_rows": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "mfq_moe_combine": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "mfq_fp8_gemm_grouped": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _i, _vp],
}
_bound = False


def _lib():
    global _bound
    L = lib()
    if not _bound:
        for name, sig in _SIGS.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = sig, C.c_int
        _bound = True
    return L


@dataclass
class RoutePlan:
    offsets: torch.Tensor  # [n_local + 1] int32
    dest: torch.Tensor  # [T, K] int32 sorted row (-1: expert not local)
    src_token: torch.Tensor  # [T*K] int32
    tile_map: torch.Tensor  # [map_cap, 2] int32
    totals: torch.Tensor  # [2] int32: rows, tiles
    token_tile: int
    max_rows: int
    n_local: int


def router_topk(x: torch.Tensor, w: torch.Tensor, k: int, *, bias: torch.Tensor | None = None, sigmoid: bool = False,
                norm_topk: bool = True, scale: float = 1.0, n_group: int = 1, topk_group: int = 1,
                want_scores: bool = False):
    t, h = x.shape
    e = w.shape[0]
    ids = torch.empty((t, k), dtype=torch.int32, device=x.device)
    wt = torch.empty((t, k), dtype=torch.float32, device=x.device)
    scores = torch.empty((t, e), dtype=torch.float32, device=x.device) if want_scores else None
    logits = torch.empty((t, e), dtype=torch.float32, device=x.device) if h % 32 == 0 else None
    rc = _lib().mfq_moe_router_topk(ptr(x), ptr(w), ptr(bias), ptr(ids), ptr(wt), ptr(scores), ptr(logits), t, h, e, k, int(sigmoid),
                                    int(norm_topk), float(scale), n_group, topk_group, stream_ptr())
    check(rc, "moe_router_topk")
    return (ids, wt, scores) if want_scores else (ids, wt)


def plan_routes(topk_ids: torch.Tensor, e_lo: int, e_hi: int, token_tile: int | None = None) -> RoutePlan:
    t, k = topk_ids.shape
    dev = topk_ids.device
    n_local = e_hi - e_lo
    bt = token_tile or K._token_tile(max(1, (t * k) // max(1, n_local)))
    # tiles = sum over non-empty experts of ceil(rows / tile): at most one per route, and at most one partial tile per expert
    map_cap = min(t * k, math.ceil(t * k / bt) + min(n_local, t * k))
    plan = RoutePlan(torch.empty(n_local + 1, dtype=torch.int32, device=dev),
                     torch.empty((t, k), dtype=torch.int32, device=dev), torch.empty(t * k, dtype=torch.int32, device=dev),
                     torch.empty((map_cap, 2), dtype=torch.int32, device=dev), torch.empty(2, dtype=torch.int32, device=dev),
                     bt, t * k, n_local)
    rc = _lib().mfq_moe_plan(ptr(topk_ids), t, k, e_lo, e_hi, bt, ptr(plan.offsets), ptr(plan.dest), ptr(plan.src_token),
                             ptr(plan.tile_map), map_cap, ptr(plan.totals), stream_ptr())
    check(rc, "moe_plan")
    return plan


def gather_rows(x_q: torch.Tensor, x_s: torch.Tensor, plan: RoutePlan):
    h = x_q.shape[1]
    out_q = torch.empty((plan.max_rows, h), dtype=x_q.dtype, device=x_q.device)
    out_s = torch.empty(plan.max_rows, dtype=torch.float32, device=x_q.device)
    check(_lib().mfq_moe_gather_rows(ptr(x_q), ptr(x_s), ptr(plan.src_token), ptr(plan.totals), ptr(out_q), ptr(out_s),
                                     plan.max_rows, h, stream_ptr()), "moe_gather_rows")
    return out_q, out_s


# Above this many routes per step the expert tiles stop being latency-bound and the tcgen05 grouped GEMM streams the
# weights faster (measured on the 512-expert hybrid: 640 routes -> 27 ms / step with the GEMM, 31 ms with the GEMV).
GEMV_MAX_ROUTES = 256


def grouped_gemv_ok(plan: RoutePlan, n: int) -> bool:
    """Decode-sized steps (a handful of rows per expert) take the weight-streaming kernel (no TMA / TMEM set-up)."""
    return plan.token_tile == 16 and n % 16 == 0 and plan.max_rows <= GEMV_MAX_ROUTES and K.gemv_enabled()


def fp8_gemm_grouped(x_q: torch.Tensor, x_s: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor, plan: RoutePlan,
                     gather: bool = False):
    """``w [E_local, N, K]`` E4M3, ``w_scale [E_local, N/128, K/128]``; rows of ``x_q`` are expert-sorted -- or, with
    ``gather`` (weight-streaming kernel only), the unsorted token rows, read through the plan's row -> token map."""
    k = x_q.shape[1]
    rows = plan.max_rows if gather else x_q.shape[0]
    e, n, _ = w.shape
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=x_q.device)
    if grouped_gemv_ok(plan, n):
        rc = lib().mfq_fp8_gemv_grouped(ptr(w), ptr(w_scale), ptr(x_q), ptr(x_s), ptr(out), n, k, ptr(plan.tile_map),
                                        plan.tile_map.shape[0], ptr(plan.offsets), ptr(plan.src_token) if gather else None,
                                        stream_ptr())
        check(rc, "fp8_gemv_grouped")
        return out
    assert not gather
    ws = Workspace.get(x_q.device)
    rc = _lib().mfq_fp8_gemm_grouped(ptr(w), ptr(w_scale), ptr(x_q), ptr(x_s), ptr(out), ptr(ws.status), rows, n, k, e,
                                     ptr(plan.tile_map), ptr(plan.offsets), plan.tile_map.shape[0], plan.token_tile,
                                     stream_ptr())
    check(rc, "fp8_gemm_grouped")
    return out


def combine(y: torch.Tensor, plan: RoutePlan, topk_w: torch.Tensor, base: torch.Tensor | None,
            extra: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    t, k = plan.dest.shape
    h = y.shape[1]
    out = torch.empty((t, h), dtype=torch.bfloat16, device=y.device) if out is None else out
    check(_lib().mfq_moe_combine(ptr(y), ptr(plan.dest), ptr(topk_w), ptr(base), ptr(extra), ptr(out), t, h, k,
                                 stream_ptr()), "moe_combine")
    return out


def moe_ffn_fp8(x_q, x_s, topk_ids, topk_w, gate_up, gate_up_scale, down, down_scale, *, e_lo: int = 0,
                base: torch.Tensor | None = None, extra: torch.Tensor | None = None, out=None) -> torch.Tensor:
    """Routed experts of one layer for this rank's experts ``[e_lo, e_lo + E_local)``; returns
    ``base + extra + sum_k w * expert_k(x)`` (only local experts contribute)."""
    plan = plan_routes(topk_ids, e_lo, e_lo + gate_up.shape[0])
    if grouped_gemv_ok(plan, gate_up.shape[1]):
        gu = fp8_gemm_grouped(x_q, x_s, gate_up, gate_up_scale, plan, gather=True)  # the gather is folded into the loads
    else:
        xq_s, xs_s = gather_rows(x_q, x_s, plan)
        gu = fp8_gemm_grouped(xq_s, xs_s, gate_up, gate_up_scale, plan)
    hq, hs = K.silu_mul_quant(gu)
    y = fp8_gemm_grouped(hq, hs, down, down_scale, plan)
    return combine(y, plan, topk_w, base, extra, out)

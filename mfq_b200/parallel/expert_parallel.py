"""Expert parallelism with token dispatch / combine fused into peer-memory kernels.

Tokens and experts are both sharded over the ``W`` ranks.  :meth:`ExpertParallel.dispatch` stores each token once per
destination rank straight into that rank's receive table (no permute pass, no size exchange); the receive table then
looks like a local batch with ``-1`` expert ids in its unused slots, so the ordinary route plan and grouped FP8 GEMMs
run over it; :meth:`ExpertParallel.combine` sums every received token's expert outputs with its routing weights,
stores the row into the source rank's return table and the source adds the returned rows to its residual.
``moe_ffn`` strings the steps together for one layer.  With ``group=None`` the same kernels run on a single GPU
(world 1), which is how they are unit-tested without a second device.

:class:`NcclExpertParallel` is the library baseline for A/B timing: torch sort/permute + ``all_to_all_single`` both
ways.  The reference has no all-to-all; it broadcasts tokens to every GPU and reduces partial outputs to a primary GPU
(``cpp_runtime/backends/cuda/core/ffn.cpp:201-300``).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops import moe as moe_ops
from ..ops.lib import Workspace, check, lib, ptr, stream_ptr
from .peer_memory import PeerBuffer

_vp, _i = C.c_void_p, C.c_int
_TABLES = 7
_SIG_DISPATCH = [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i] + [_vp] * _TABLES + [_vp, _vp, _vp]
_SIG_COMBINE = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i] + [_vp] * _TABLES + [_vp, _vp, _vp]


class _LocalBuffer:
    """Single-rank stand-in for :class:`PeerBuffer` (a zeroed device allocation and a one-entry pointer table)."""

    def __init__(self, nbytes: int, device: torch.device) -> None:
        self.mem = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=device)
        self.ptrs = [self.mem.data_ptr()]

    def table(self):
        return (C.c_void_p * 1)(*self.ptrs)


@dataclass
class Received:
    """What :meth:`ExpertParallel.dispatch` leaves on this rank: views of the receive table (``W * cap`` slots)."""

    x_q: torch.Tensor  # [W*cap, H] fp8
    x_scale: torch.Tensor  # [W*cap] fp32
    ids: torch.Tensor  # [W*cap, K] int32, -1 in unused slots
    weights: torch.Tensor  # [W*cap, K] fp32
    send_slot: torch.Tensor  # [T, W] int32: slot of my token t on rank r, -1 if not sent there
    total: torch.Tensor  # [1] int32: rows received
    tokens: int
    cap: int


class ExpertParallel:
    def __init__(self, group, device: torch.device, *, num_experts: int, top_k: int, hidden: int, max_tokens: int) -> None:
        """``max_tokens``: the most tokens any one rank dispatches per call (sizes the tables: W * max_tokens slots)."""
        self.group, self.device = group, torch.device(device)
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        if num_experts % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.e_per, self.k, self.h, self.cap_max = num_experts // self.world, top_k, hidden, max_tokens
        slots = self.world * max_tokens

        def buf(nbytes):
            return PeerBuffer(group, nbytes, self.device) if group is not None else _LocalBuffer(nbytes, self.device)

        self._bufs = [buf(slots * hidden), buf(slots * 4), buf(slots * top_k * 4), buf(slots * top_k * 4),
                      buf(max(256, self.world * 4)), buf(max(256, 2 * self.world * 4)), buf(slots * hidden * 2)]
        self._tables = [b.table() for b in self._bufs]
        self._words = torch.zeros(2 + self.world, dtype=torch.int32, device=self.device)
        L = lib()
        L.mfq_moe_dispatch.argtypes, L.mfq_moe_dispatch.restype = _SIG_DISPATCH, C.c_int
        L.mfq_moe_combine_a2a.argtypes, L.mfq_moe_combine_a2a.restype = _SIG_COMBINE, C.c_int
        self._views: dict[int, tuple] = {}

    def _own(self, i: int, dtype: torch.dtype, shape) -> torch.Tensor:
        """Typed view of this rank's own allocation ``i`` (a zero-copy alias of the peer-mapped memory)."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        b = self._bufs[i]
        mem = b.mem if isinstance(b, _LocalBuffer) else b.local_tensor()
        return mem[:nbytes].view(dtype).view(shape)

    def dispatch(self, x_q: torch.Tensor, x_scale: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                 cap: int | None = None) -> Received:
        """Send my ``T`` tokens to the ranks that own their experts and wait for everybody's.  ``cap`` (same on all
        ranks, >= every rank's T) is the slot count per source this call; it defaults to the table capacity."""
        t, h = x_q.shape
        cap = self.cap_max if cap is None else cap
        if t > cap or cap > self.cap_max or h != self.h or ids.shape != (t, self.k):
            raise ValueError("dispatch: token count, hidden size or top-k does not fit the tables")
        send_slot = torch.empty((max(t, 1), self.world), dtype=torch.int32, device=self.device)
        total = torch.empty(1, dtype=torch.int32, device=self.device)
        ws = Workspace.get(self.device)
        rc = lib().mfq_moe_dispatch(ptr(x_q), ptr(x_scale), ptr(ids), ptr(weights), t, h, ptr(send_slot), ptr(total),
                                    self.world, self.rank, self.k, cap, self.e_per, *self._tables, ptr(self._words),
                                    ptr(ws.status), stream_ptr())
        check(rc, "moe_dispatch", 2)
        slots = self.world * cap
        views = self._views.get(cap)
        if views is None:
            views = self._views[cap] = (self._own(0, torch.float8_e4m3fn, (slots, h)), self._own(1, torch.float32, (slots,)),
                                        self._own(2, torch.int32, (slots, self.k)), self._own(3, torch.float32, (slots, self.k)))
        return Received(*views, send_slot, total, t, cap)

    def combine(self, y: torch.Tensor, plan: moe_ops.RoutePlan, recv: Received, base: torch.Tensor | None = None,
                extra: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """``out[t] = base[t] + extra[t] + sum_k w[t,k] * expert_k(x[t])`` for my ``T`` tokens; ``y`` holds this rank's
        expert outputs in route-plan order."""
        h = y.shape[1]
        out = torch.empty((recv.tokens, h), dtype=torch.bfloat16, device=self.device) if out is None else out
        ws = Workspace.get(self.device)
        rc = lib().mfq_moe_combine_a2a(ptr(y), ptr(plan.dest), ptr(recv.send_slot), ptr(base), ptr(extra), ptr(out),
                                       recv.tokens, h, self.world, self.rank, self.k, recv.cap, self.e_per, *self._tables,
                                       ptr(self._words), ptr(ws.status), stream_ptr())
        check(rc, "moe_combine_a2a", 2)
        return out

    def moe_ffn(self, x_q, x_scale, ids, weights, gate_up, gate_up_scale, down, down_scale, *, base=None, extra=None,
                out=None, cap: int | None = None) -> torch.Tensor:
        """One routed-experts layer for token-sharded input: dispatch -> grouped GEMMs on my experts -> combine."""
        recv = self.dispatch(x_q, x_scale, ids, weights, cap)
        e_lo = self.rank * self.e_per
        plan = moe_ops.plan_routes(recv.ids, e_lo, e_lo + self.e_per)
        xq_s, xs_s = moe_ops.gather_rows(recv.x_q, recv.x_scale, plan)
        gu = moe_ops.fp8_gemm_grouped(xq_s, xs_s, gate_up, gate_up_scale, plan)
        hq, hs = K.silu_mul_quant(gu)
        y = moe_ops.fp8_gemm_grouped(hq, hs, down, down_scale, plan)
        return self.combine(y, plan, recv, base, extra, out)


class NcclExpertParallel:
    """Library baseline: sort by destination rank, exchange sizes, ``all_to_all_single`` there and back."""

    def __init__(self, group, device, *, num_experts: int, top_k: int, hidden: int, max_tokens: int) -> None:
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.e_per, self.k, self.h = num_experts // self.world, top_k, hidden

    def dispatch(self, x_q, x_scale, ids, weights):
        t = x_q.shape[0]
        owner = torch.div(ids, self.e_per, rounding_mode="floor")  # [T, K]
        goes = torch.zeros((t, self.world), dtype=torch.bool, device=self.device).scatter_(1, owner.long(), True)
        tok, dst = goes.nonzero(as_tuple=True)
        order = torch.argsort(dst, stable=True)
        tok, dst = tok[order], dst[order]
        send_counts = torch.bincount(dst, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        n = sum(rc)

        def exchange(rows):
            out = torch.empty((n,) + rows.shape[1:], dtype=rows.dtype, device=self.device)
            dist.all_to_all_single(out, rows.contiguous(), rc, sc, group=self.group)
            return out

        rx = exchange(x_q[tok].view(torch.uint8)).view(torch.float8_e4m3fn)
        return rx, exchange(x_scale[tok]), exchange(ids[tok]), exchange(weights[tok]), (tok, sc, rc, t)

    def combine(self, y_tokens, ctx, base=None):
        """``y_tokens [n_received, H]`` bf16: the weighted expert sum of every received token."""
        tok, sc, rc, t = ctx
        back = torch.empty((sum(sc), y_tokens.shape[1]), dtype=y_tokens.dtype, device=self.device)
        dist.all_to_all_single(back, y_tokens.contiguous(), sc, rc, group=self.group)
        out = torch.zeros((t, y_tokens.shape[1]), dtype=torch.float32, device=self.device) if base is None else base.float().clone()
        out.index_add_(0, tok, back.float())
        return out.to(torch.bfloat16)

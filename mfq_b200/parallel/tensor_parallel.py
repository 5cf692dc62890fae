"""Tensor parallelism over the GPUs of one node: symmetric ranks, collectives fused into the kernels.

Every rank owns 1/W of the attention heads and of the MLP intermediate; the residual stream is replicated.
Row-parallel projections (``o_proj``, ``down``) run :func:`mfq_fp8_gemm_allreduce`, whose epilogue exchanges the
partial tiles through peer-mapped memory and sums them in rank order (bit-identical on all ranks); the sampled
token comes from a vocabulary-sharded arg-max that exchanges 8 bytes per rank and row.  The reference instead
broadcasts activations from, and reduces partial outputs to, one primary GPU through NCCL
(``cpp_runtime/backends/cuda/ops/quant_linear.cpp:622-761``).  :class:`NcclTensorParallel` is that style of
baseline (library collectives after an unfused GEMM), kept for A/B measurements.
"""

from __future__ import annotations

import ctypes as C
import math

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops.lib import Workspace, check, lib, ptr, stream_ptr
from .peer_memory import PeerBuffer


class _ReduceContext:
    """Peer buffers of one (token tile, N, token-tile count) geometry."""

    def __init__(self, tp: "TensorParallel", bt: int, n: int, t_tiles: int) -> None:
        self.tiles = math.ceil(n / 128) * t_tiles
        self.half_elems = self.tiles * bt * 128
        self.partials = PeerBuffer(tp.group, 2 * self.half_elems * 4, tp.device)
        self.flags = PeerBuffer(tp.group, max(256, self.tiles * 4), tp.device)
        self.expected = torch.zeros(self.tiles, dtype=torch.int32, device=tp.device)
        self.buf_table = self.partials.table()
        self.flag_table = self.flags.table()


class FusedStream:
    """Peer-mapped buffers of the decode-sized residual stream of one hidden size, and the fused
    all-reduce + residual + RMSNorm + FP8-quantization kernel over them (``ops/csrc/tp_reduce.cu``).

    ``partial_out(m)`` is where a row-parallel GEMM writes this rank's bf16 partial (two halves used alternately);
    :meth:`reduce` then sums all ranks' partials into the residual stream ``h`` and, given norm weights, leaves the
    next GEMM's input ``(xq, xs)``.  With ``h`` inside this object's own buffer (:meth:`h_rows`) and enough rows the
    two-shot mode is used: each rank finishes 1/W of the rows and pushes them to the others."""

    TWO_SHOT_MIN_ROWS = 64

    def __init__(self, tp: "TensorParallel", hidden: int, rows_cap: int = 1024) -> None:
        self.tp, self.hidden, self.rows_cap = tp, hidden, rows_cap
        g, dev = tp.group, tp.device
        self.partials = PeerBuffer(g, 2 * rows_cap * hidden * 2, dev)
        self.h = PeerBuffer(g, rows_cap * hidden * 2, dev)
        self.xq = PeerBuffer(g, rows_cap * hidden, dev)
        self.xs = PeerBuffer(g, rows_cap * 4, dev)
        self.flags = PeerBuffer(g, 256, dev)
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)
        self._partial_t = self.partials.local_tensor().view(torch.bfloat16).view(2, rows_cap, hidden)
        self._h_t = self.h.local_tensor().view(torch.bfloat16).view(rows_cap, hidden)
        self._xq_t = self.xq.local_tensor().view(FP8_DTYPE).view(rows_cap, hidden)
        self._xs_t = self.xs.local_tensor().view(torch.float32)
        self._tables = (self.partials.table(), self.h.table(), self.xq.table(), self.xs.table(), self.flags.table())
        self.half = 0

    def h_rows(self, m: int) -> torch.Tensor:
        """The first ``m`` rows of the peer-mapped residual stream (keep the model's ``h`` here to enable two-shot)."""
        return self._h_t[:m]

    def partial_out(self, m: int) -> torch.Tensor:
        return self._partial_t[self.half, :m]

    def reduce(self, m: int, h: torch.Tensor, norm_w: torch.Tensor | None, eps: float = 0.0, add_residual: bool = True):
        """``h += sum_r partial_r`` (the partials of the half :meth:`partial_out` last returned); with ``norm_w`` also
        returns ``(xq, xs) = quant(rmsnorm(h) * norm_w)``.  ``h`` may be any ``[m, hidden]`` bf16 tensor of this rank;
        rows inside :meth:`h_rows` allow the two-shot mode."""
        tp = self.tp
        own = h.data_ptr() == self._h_t.data_ptr()
        two_shot = int(own and m >= self.TWO_SHOT_MIN_ROWS and m >= 2 * tp.world)
        tables = self._tables
        if not own:  # one-shot only: the residual stream is read and written locally at the caller's address
            h_table = (C.c_void_p * tp.world)(*[h.data_ptr()] * tp.world)
            tables = (tables[0], h_table, *tables[2:])
        fn = lib().mfq_tp_reduce_norm_quant
        fn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6 + \
                      [C.c_int, C.c_void_p, C.c_void_p]
        ws = Workspace.get(tp.device)
        rc = fn(m, self.hidden, self.half, ptr(norm_w), float(eps), two_shot, int(add_residual), tp.world, tp.rank, *tables,
                ptr(self.state), self.rows_cap, ptr(ws.status), stream_ptr())
        check(rc, "tp_reduce_norm_quant")
        self.half ^= 1
        if norm_w is None:
            return h, None, None
        return h, self._xq_t[:m], self._xs_t[:m]


FP8_DTYPE = torch.float8_e4m3fn


class TensorParallel:
    def __init__(self, group, device: torch.device, max_rows: int = 8192) -> None:
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._ctx: dict[tuple[int, int, int], _ReduceContext] = {}
        self._streams: dict[int, FusedStream] = {}
        self.rows_cap = max_rows
        self.fused = True  # False: the GEMM-epilogue exchange (per-tile flags) also for decode-sized batches
        self._slots = PeerBuffer(group, 2 * self.world * max_rows * 8, device)
        self._slot_flags = PeerBuffer(group, max_rows * 4, device)
        self._slot_expected = torch.zeros(max_rows, dtype=torch.int32, device=device)

    def stream(self, hidden: int) -> FusedStream:
        """The fused-reduce buffers of one hidden size (created on first use: a collective call)."""
        st = self._streams.get(hidden)
        if st is None:
            st = self._streams[hidden] = FusedStream(self, hidden)
        return st

    def begin_step(self) -> None:
        """Call at the start of every forward pass: a device-side barrier of all ranks, after which the fused reduce
        starts again at half 0 of its partial buffers.  The halves are chosen on the host (and frozen into captured
        graphs), so without this two consecutive passes could use the same half back to back."""
        self.barrier()
        for st in self._streams.values():
            st.half = 0

    def row_parallel_fused(self, lin, x_q: torch.Tensor, x_scale: torch.Tensor, h: torch.Tensor,
                           norm_w: torch.Tensor | None = None, eps: float = 0.0):
        """``h += all_reduce(x_q @ lin^T)``, then ``(xq, xs) = quant(rmsnorm(h) * norm_w)`` for the next GEMM: the local
        GEMM writes its bf16 partial into peer-mapped memory and ONE kernel does the exchange, the residual add, the
        norm and the quantization.  Returns ``(h, xq, xs)`` (the latter None without ``norm_w``).  ``m`` must not
        exceed the stream's row capacity."""
        m = x_q.shape[0]
        st = self.stream(lin.q.shape[0])
        K.fp8_gemm(x_q, x_scale, lin.q, lin.scale, out=st.partial_out(m))
        return st.reduce(m, h, norm_w, eps)

    def stream_rows(self, hidden: int, rows: int) -> torch.Tensor:
        """``[rows, hidden]`` bf16 view of the peer-mapped residual stream (where the model keeps ``h``)."""
        return self.stream(hidden).h_rows(rows)

    def fused_rows(self, hidden: int) -> int:
        """Largest row count the fused reduce of this hidden size accepts."""
        return self.stream(hidden).rows_cap

    def row_parallel_linear(self, lin, x_q: torch.Tensor, x_scale: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """``h += all_reduce(x_q @ lin^T)`` in place; ``x_q`` holds this rank's input shard."""
        m, k = x_q.shape
        n = lin.q.shape[0]
        if m <= self.fused_rows(n) and self.fused:
            return self.row_parallel_fused(lin, x_q, x_scale, h)[0]
        if m % (self.world * 128) == 0:
            # wide batches: two-shot (reduce-scatter in the GEMM epilogue, then all-gather of the bf16 rows) moves
            # 2(W-1)/W of the output per rank instead of the (W-1)x of the one-shot exchange
            rows = m // self.world
            shard = self.gemm_reduce_scatter(lin, x_q, x_scale, h[self.rank * rows:(self.rank + 1) * rows])
            return self.allgather_rows(shard, out=h)
        bt = K._token_tile(m)
        key = (bt, n, math.ceil(m / bt))
        ctx = self._ctx.get(key)
        if ctx is None:
            ctx = self._ctx[key] = _ReduceContext(self, *key)
        ws = Workspace.get(self.device)
        rc = lib().mfq_fp8_gemm_allreduce(
            ptr(lin.q), ptr(lin.scale), ptr(x_q), ptr(x_scale), ptr(h), ptr(h), ptr(ws.splitk), ws.splitk.numel(),
            ptr(ws.counters), ws.counters.numel(), ptr(ws.status), m, n, k, bt, K.pick_splits(m, n, k), self.world,
            self.rank, ctx.buf_table, ctx.flag_table, ptr(ctx.expected), ctx.half_elems, 0, stream_ptr())
        check(rc, "fp8_gemm_allreduce")
        return h

    def gemm_reduce_scatter(self, lin, x_q: torch.Tensor, x_scale: torch.Tensor, residual_shard: torch.Tensor | None = None,
                            token_tile: int = 128) -> torch.Tensor:
        """Row-parallel GEMM whose epilogue reduce-scatters over token rows: returns this rank's ``[M/W, N]`` shard of
        ``sum_r x_r @ lin_r^T (+ residual_shard)``.  ``M`` must be a multiple of ``W * token_tile``."""
        m, k = x_q.shape
        n = lin.q.shape[0]
        key = ("rs", token_tile, n, math.ceil(m / token_tile))
        ctx = self._ctx.get(key)
        if ctx is None:
            ctx = self._ctx[key] = _ReduceContext(self, token_tile, n, math.ceil(m / token_tile))
        out = torch.empty((m // self.world, n), dtype=torch.bfloat16, device=self.device)
        ws = Workspace.get(self.device)
        rc = lib().mfq_fp8_gemm_allreduce(
            ptr(lin.q), ptr(lin.scale), ptr(x_q), ptr(x_scale), ptr(out), ptr(residual_shard), ptr(ws.splitk),
            ws.splitk.numel(), ptr(ws.counters), ws.counters.numel(), ptr(ws.status), m, n, k, token_tile, 1, self.world,
            self.rank, ctx.buf_table, ctx.flag_table, ptr(ctx.expected), ctx.half_elems, 1, stream_ptr())
        check(rc, "fp8_gemm_reduce_scatter")
        # every rank's pushes are complete once its GEMM kernel is: meet on the stream, then sum the owned tiles
        self.barrier()
        fn = lib().mfq_rs_reduce
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t,
                       C.c_void_p]
        check(fn(ptr(out), ptr(residual_shard), m, n, token_tile, self.world, self.rank, ctx.buf_table, ptr(ctx.expected),
                 ctx.half_elems, stream_ptr()), "rs_reduce")
        return out

    def allgather_gemm(self, lin, xq_shard: torch.Tensor, xs_shard: torch.Tensor, token_tile: int = 128,
                       push_ctas: int | None = None) -> torch.Tensor:
        """Column-parallel GEMM over token-sharded input: gathers the shards through peer memory inside the kernel
        and returns ``[M, N_local]``."""
        ms, k = xq_shard.shape
        if push_ctas is None:  # one push block per 64 KB of shard, at most 32: tiny shards are latency-, not bandwidth-bound
            push_ctas = max(4, min(32, (ms * k) // 65536))
        m = ms * self.world
        n = lin.q.shape[0]
        key = ("ag", m, k)
        ctx = self._ctx.get(key)
        if ctx is None:
            class _AgCtx:
                pass
            ctx = _AgCtx()
            ctx.x = PeerBuffer(self.group, 2 * m * k, self.device)
            ctx.xs = PeerBuffer(self.group, 2 * m * 4, self.device)
            ctx.flags = PeerBuffer(self.group, 256, self.device)
            ctx.words = torch.zeros(16, dtype=torch.int32, device=self.device)  # epoch, then one push counter per destination
            ctx.tables = (ctx.x.table(), ctx.xs.table(), ctx.flags.table())
            self._ctx[key] = ctx
        out = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
        ws = Workspace.get(self.device)
        rc = lib().mfq_fp8_gemm_allgather(ptr(lin.q), ptr(lin.scale), ptr(xq_shard), ptr(xs_shard), ptr(out), ptr(ws.status),
                                          m, n, k, token_tile, self.world, self.rank, *ctx.tables, ctx.words.data_ptr(),
                                          ctx.words.data_ptr() + 4, push_ctas, stream_ptr())
        check(rc, "fp8_gemm_allgather", 2)
        return out

    def allgather_rows(self, shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``[rows, width]`` per rank -> ``[W * rows, width]`` in rank order on every rank (peer-memory push)."""
        shard = shard.contiguous()
        nbytes = shard.numel() * shard.element_size()
        half = self.world * nbytes
        key = ("gather", half)
        ctx = self._ctx.get(key)
        if ctx is None:
            class _GatherCtx:
                pass
            ctx = _GatherCtx()
            ctx.bufs = PeerBuffer(self.group, 2 * half, self.device)
            ctx.flags = PeerBuffer(self.group, 256, self.device)
            ctx.words = torch.zeros(2, dtype=torch.int32, device=self.device)
            ctx.tables = (ctx.bufs.table(), ctx.flags.table())
            self._ctx[key] = ctx
        if out is None:
            out = torch.empty((self.world * shard.shape[0],) + tuple(shard.shape[1:]), dtype=shard.dtype, device=self.device)
        fn = lib().mfq_allgather_rows
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                       C.c_longlong, C.c_void_p, C.c_void_p]
        ws = Workspace.get(self.device)
        check(fn(ptr(shard), ptr(out), nbytes, self.world, self.rank, *ctx.tables, ptr(ctx.words), half, ptr(ws.status),
                 stream_ptr()), "allgather_rows", 2)
        return out

    def broadcast_rows(self, h: torch.Tensor, src: int) -> torch.Tensor:
        """Layer placement hand-off: every rank receives rank ``src``'s rows (in place; a few KB per step, so the
        library broadcast over NVLink is used -- it is capturable in a CUDA graph)."""
        import torch.distributed as dist
        dist.broadcast(h, src=dist.get_global_rank(self.group, src) if hasattr(dist, "get_global_rank") else src, group=self.group)
        return h

    def barrier(self) -> None:
        """Device-side barrier of all ranks on the current stream (bounded wait, no host synchronisation)."""
        if not hasattr(self, "_bar"):
            self._bar = (PeerBuffer(self.group, 256, self.device), torch.zeros(1, dtype=torch.int32, device=self.device))
        flags, expected = self._bar
        ws = Workspace.get(self.device)
        check(lib().mfq_peer_barrier(self.world, self.rank, flags.table(), ptr(expected), ptr(ws.status), stream_ptr()), "peer_barrier")

    def argmax(self, logits_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        b, v = logits_shard.shape
        out = torch.empty(b, dtype=torch.int32, device=self.device) if out is None else out
        ws = Workspace.get(self.device)
        rc = lib().mfq_argmax_allgather(ptr(logits_shard), ptr(out), b, v, logits_shard.stride(0), self.rank * v,
                                        self.world, self.rank, self._slots.table(), self._slot_flags.table(),
                                        ptr(self._slot_expected), self.rows_cap, ptr(ws.status), stream_ptr())
        check(rc, "argmax_allgather")
        return out

    def allreduce_rows(self, partial: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """``h += sum over ranks of partial`` in place (one fused kernel over peer memory)."""
        rows, width = partial.shape
        if self.fused and rows <= self.fused_rows(width):
            st = self.stream(width)
            st.partial_out(rows).copy_(partial)
            return st.reduce(rows, h, None)[0]
        key = ("rows", width)
        ctx = self._ctx.get(key)
        if ctx is None:
            cap = self.rows_cap

            class _RowCtx:
                pass
            ctx = _RowCtx()
            ctx.bufs = PeerBuffer(self.group, 2 * cap * width * 2, self.device)
            ctx.flags = PeerBuffer(self.group, cap * 4, self.device)
            ctx.expected = torch.zeros(cap, dtype=torch.int32, device=self.device)
            ctx.buf_table, ctx.flag_table = ctx.bufs.table(), ctx.flags.table()
            self._ctx[key] = ctx
        ws = Workspace.get(self.device)
        fn = lib().mfq_allreduce_rows
        fn.argtypes = [C.c_void_p] * 3 + [C.c_int] * 4 + [C.c_void_p] * 3 + [C.c_int, C.c_void_p, C.c_void_p]
        rc = fn(ptr(partial), ptr(h), ptr(h), rows, width, self.world, self.rank, ctx.buf_table, ctx.flag_table,
                ptr(ctx.expected), self.rows_cap, ptr(ws.status), stream_ptr())
        check(rc, "allreduce_rows")
        return h

    def gather_columns(self, shard: torch.Tensor) -> torch.Tensor:
        """Full ``[rows, W * cols]`` matrix from column shards (library all-gather; used off the hot path)."""
        parts = [torch.empty_like(shard) for _ in range(self.world)]
        dist.all_gather(parts, shard.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)


class NcclTensorParallel(TensorParallel):
    """Baseline: unfused GEMM followed by NCCL all-reduce / all-gather (what a library-only port would do)."""

    def __init__(self, group, device, max_rows: int = 8192) -> None:
        super().__init__(group, device, max_rows)
        self.fused = False

    def begin_step(self) -> None:
        pass

    def allreduce_rows(self, partial, h):
        total = partial.float()
        dist.all_reduce(total, group=self.group)
        h.copy_((total + h.float()).to(torch.bfloat16))
        return h

    def row_parallel_linear(self, lin, x_q, x_scale, h):
        partial = K.fp8_gemm(x_q, x_scale, lin.q, lin.scale).float()
        dist.all_reduce(partial, group=self.group)
        h.copy_((partial + h.float()).to(torch.bfloat16))
        return h

    def argmax(self, logits_shard, out=None):
        full = self.gather_columns(logits_shard)
        res = K.argmax(full)
        if out is not None:
            out.copy_(res)
            return out
        return res

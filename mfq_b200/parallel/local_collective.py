"""In-process ranks: the model's collective interface over threads of one process, for CPU tensors.

``LocalGroup(world)`` hands out one :class:`LocalCollective` per rank; the ranks run the same model code in threads and
meet at a barrier inside every collective call, exchanging tensors through a shared list.  It mirrors what the fused
GPU kernels compute (``row_parallel_linear`` = partial product on every rank, summed, plus the residual; ``argmax`` over
vocabulary shards with the lowest global index winning ties) so tensor- and expert-parallel model code can be checked
against the single-rank result without GPUs.  Reference: the reference validates its TP/EP graph code on one device the
same way (``docs/runtime/support.md``: tensor/expert parallel paths are host-validated).
"""

from __future__ import annotations

import threading

import torch


class LocalGroup:
    def __init__(self, world: int, timeout: float = 120.0) -> None:
        self.world = world
        self.slots: list = [None] * world
        self.barrier = threading.Barrier(world, timeout=timeout)

    def member(self, rank: int) -> "LocalCollective":
        return LocalCollective(self, rank)

    def run(self, fn) -> list:
        """``fn(rank, collective)`` on every rank in its own thread; returns the results in rank order and re-raises
        the first failure (a failed rank breaks the barrier, so the others stop instead of waiting for it)."""
        out, errs = [None] * self.world, []

        def body(r):
            try:
                out[r] = fn(r, self.member(r))
            except BaseException as exc:  # noqa: BLE001 - reported to the caller below
                errs.append(exc)
                self.barrier.abort()

        threads = [threading.Thread(target=body, args=(r,)) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        real = [e for e in errs if not isinstance(e, threading.BrokenBarrierError)]
        if real or errs:
            raise (real or errs)[0]
        return out


class LocalCollective:
    def __init__(self, group: LocalGroup, rank: int) -> None:
        self.group, self.rank, self.world = group, rank, group.world

    def _exchange(self, value):
        g = self.group
        g.slots[self.rank] = value
        g.barrier.wait()
        everyone = list(g.slots)
        g.barrier.wait()  # nobody overwrites a slot before all have read it
        return everyone

    # ---- the interface the models use ------------------------------------------------------------------------------
    def row_parallel_linear(self, lin, *args) -> torch.Tensor:
        *x_in, h = args
        parts = self._exchange(lin(*x_in).float())
        total = h.float()
        for p in parts:  # rank order: every rank computes the same sum
            total = total + p
        h.copy_(total.to(h.dtype))
        return h

    # the fused reduce of the GPU path (ops/csrc/tp_reduce.cu): bf16 partials, summed in rank order in fp32, plus the
    # residual, stored as bf16; then RMSNorm + FP8 row quantization of the stored rows
    fused = True

    def begin_step(self) -> None:
        pass

    def fused_rows(self, hidden: int) -> int:
        return 1024

    def stream_rows(self, hidden: int, rows: int) -> torch.Tensor:
        return torch.empty((rows, hidden), dtype=torch.bfloat16)

    def row_parallel_fused(self, lin, x_q, x_scale, h, norm_w=None, eps: float = 0.0):
        from ..ops import reference as ref
        parts = self._exchange(lin(x_q, x_scale).to(torch.bfloat16).float())
        total = torch.zeros_like(parts[0])
        for p in parts:
            total = total + p
        h.copy_((total + h.float()).to(h.dtype))
        if norm_w is None:
            return h, None, None
        q, s, _, _ = ref.rmsnorm_quant(h, norm_w, eps)
        return h, q, s

    def allreduce_rows(self, partial: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        parts = self._exchange(partial.float())
        total = h.float()
        for p in parts:
            total = total + p
        h.copy_(total.to(h.dtype))
        return h

    def gather_columns(self, shard: torch.Tensor) -> torch.Tensor:
        return torch.cat(self._exchange(shard), dim=1)

    def allgather_rows(self, shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        full = torch.cat(self._exchange(shard), dim=0)
        if out is not None:
            out.copy_(full)
            return out
        return full

    def argmax(self, logits_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        v = logits_shard.shape[1]
        best = logits_shard.float().max(dim=1)
        cands = self._exchange((best.values, best.indices + self.rank * v))
        vals = torch.stack([c[0] for c in cands], 1)
        idx = torch.stack([c[1] for c in cands], 1)
        # the highest value wins; among equal values the lowest global index (ranks hold ascending index ranges)
        pick = (vals == vals.max(dim=1, keepdim=True).values).float().argmax(dim=1)
        res = idx.gather(1, pick[:, None])[:, 0].to(torch.int32)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def broadcast_rows(self, h: torch.Tensor, src: int) -> torch.Tensor:
        """Every rank gets rank ``src``'s tensor (layer placement: the stage owner hands the residual stream on)."""
        got = self._exchange(h)[src]
        return got if src == self.rank else got.clone()

    def barrier(self) -> None:
        self.group.barrier.wait()


class ProcessGroupCollective(LocalCollective):
    """The same interface across PROCESSES, over a ``torch.distributed`` group of CPU tensors (``gloo``).

    It exists so that the whole multi-rank serving path (launcher, command log, sharded checkpoint load, tensor- and
    expert-parallel model code) runs end to end on machines without GPUs; GPU ranks use the fused peer-memory
    collectives of :class:`~mfq_b200.parallel.tensor_parallel.TensorParallel` instead."""

    def __init__(self, group=None) -> None:
        import torch.distributed as dist
        self._dist, self.pg = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def _exchange(self, value):
        out = [None] * self.world
        self._dist.all_gather_object(out, value, group=self.pg)
        return out

    def barrier(self) -> None:
        self._dist.barrier(group=self.pg)

"""MoE expert residency: an HBM slot arena in front of a pinned-host tier.

Models whose routed experts exceed the GPU keep every expert in pinned host memory and only ``slots`` of them in HBM.
The grouped expert GEMMs index the ARENA (``[slots, ...]``), so routing ids are translated expert -> slot before the
route plan and no kernel changes:

    ids_slot = residency.ensure(topk_ids)        # uploads what is missing, returns slot ids (same shape)
    moe_ffn_fp8(x, xs, ids_slot, w, arena.gate_up, arena.gate_up_scale, arena.down, arena.down_scale, e_lo=0, ...)

* ``ensure`` reads the step's expert histogram on the host (one small D2H), pins the experts the step uses, evicts
  the least recently used unpinned slots for the missing ones (C++ slot book), and issues the uploads with
  ``non_blocking`` copies on a side stream; the compute stream waits on an event (stream-ordered, no spinning).
* ``rebalance`` between steps swaps cold residents for hotter absent experts (C++ ranker, exponential heat).
* When a step needs more distinct experts than there are slots it is processed in waves of at most ``slots`` experts.

Reference: the residency manager, pinned expert arena and slot book of
``cpp_runtime/backends/cuda/runtime/moe_residency_manager.*``, ``storage/moe_expert_cache*``,
``engine/include/moe_cache_policy.h``; there the device polls host-written ready flags, here readiness is an event.

Optimistic mode (``enable_optimistic``) keeps such a model inside CUDA graphs: a step translates ids through the device
slot table as it is, routes to absent experts are skipped and counted in one device word; the engine reads that word
after the step, and only when it is not zero uploads what was missing (``settle``), restores the few words of sequence
state and runs the step again -- KV rows are simply rewritten.  Nothing on the device ever waits for an upload.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import native


@dataclass
class ExpertArena:
    gate_up: torch.Tensor  # [slots, 2I, H] fp8
    gate_up_scale: torch.Tensor
    down: torch.Tensor  # [slots, H, I] fp8
    down_scale: torch.Tensor


class ExpertResidency:
    def __init__(self, gate_up: torch.Tensor, gate_up_scale: torch.Tensor, down: torch.Tensor, down_scale: torch.Tensor,
                 slots: int, device, heat_decay: float = 0.9) -> None:
        """The four tensors hold ALL experts on the host (``[E, ...]``); they are pinned when the device is a GPU."""
        self.device = torch.device(device)
        self.n = gate_up.shape[0]
        self.slots = min(slots, self.n)
        cuda = self.device.type == "cuda"
        self.host = tuple(t.contiguous().pin_memory() if cuda else t.contiguous() for t in (gate_up, gate_up_scale, down, down_scale))
        self.arena = ExpertArena(*(torch.empty((self.slots,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.device) for t in self.host))
        self.book = native.SlotBook(self.slots)
        self.slot_of = np.full(self.n, -1, dtype=np.int32)
        self.slot_of_dev = torch.full((self.n,), -1, dtype=torch.int32, device=self.device)
        self.heat = np.zeros(self.n, dtype=np.float64)
        self.decay = heat_decay
        self.copy_stream = torch.cuda.Stream(device=self.device) if cuda else None
        self.stats = {"hits": 0, "uploads": 0, "evictions": 0, "waves": 0, "upload_bytes": 0}
        self.bytes_per_expert = sum(t[0].numel() * t[0].element_size() for t in self.host)
        self.optimistic = False

    # -- uploads ------------------------------------------------------------------------------------------------
    def _upload(self, expert: int, slot: int) -> None:
        for dst, src in zip((self.arena.gate_up, self.arena.gate_up_scale, self.arena.down, self.arena.down_scale), self.host):
            dst[slot].copy_(src[expert], non_blocking=True)
        self.stats["uploads"] += 1
        self.stats["upload_bytes"] += self.bytes_per_expert

    def _make_resident(self, experts: list[int]) -> None:
        """All of ``experts`` (at most ``slots`` many) resident and pinned; uploads ordered before later compute."""
        missing = [e for e in experts if self.slot_of[e] < 0]
        for e in experts:
            if self.slot_of[e] >= 0:
                self.book.lookup(int(e))
                self.book.pin(int(e), +1)
                self.stats["hits"] += 1
        if missing:
            ctx = torch.cuda.stream(self.copy_stream) if self.copy_stream is not None else _Null()
            if self.copy_stream is not None:
                self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))  # slots may still be read
            with ctx:
                for e in missing:
                    slot, evicted = self.book.acquire(int(e))
                    if evicted is not None:
                        self.slot_of[evicted] = -1
                        self.stats["evictions"] += 1
                    self.slot_of[e] = slot
                    self.book.pin(int(e), +1)
                    self._upload(int(e), slot)
            if self.copy_stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
        self.slot_of_dev.copy_(torch.from_numpy(self.slot_of), non_blocking=True)

    def _unpin(self, experts: list[int]) -> None:
        for e in experts:
            self.book.pin(int(e), -1)

    # -- per step -----------------------------------------------------------------------------------------------
    def waves(self, topk_ids: torch.Tensor) -> list[list[int]]:
        """Experts the step uses, hottest first, cut into groups of at most ``slots``; also updates the heat."""
        flat = topk_ids.reshape(-1).cpu().numpy().astype(np.int64)
        counts = np.bincount(flat[flat >= 0], minlength=self.n)[: self.n]  # negative ids: experts of other ranks
        self.heat = self.heat * self.decay + counts
        used = [int(e) for e in np.argsort(-counts, kind="stable") if counts[e] > 0]
        return [used[i : i + self.slots] for i in range(0, len(used), self.slots)]

    def run(self, topk_ids: torch.Tensor, fn):
        """Calls ``fn(ids_slot, arena)`` once per wave and sums the results.  ``ids_slot`` has the shape of
        ``topk_ids`` with arena slots for the wave's experts and -1 elsewhere (the route plan skips -1)."""
        out = None
        for wave in self.waves(topk_ids):
            self.stats["waves"] += 1
            self._make_resident(wave)
            in_wave = torch.zeros(self.n, dtype=torch.bool, device=self.device)
            in_wave[torch.as_tensor(wave, device=self.device, dtype=torch.long)] = True
            ids = topk_ids.long().clamp(min=0)
            mine = in_wave[ids] & (topk_ids >= 0)
            ids_slot = torch.where(mine, self.slot_of_dev[ids], torch.full_like(self.slot_of_dev[ids], -1)).to(torch.int32)
            part = fn(ids_slot, self.arena)
            out = part if out is None else out + part
            self._unpin(wave)
        return out

    def warm(self, heat=None) -> list[int]:
        """Make the hottest ``slots`` experts resident before traffic arrives (``heat``: a saved profile for this
        layer; default: the heat gathered so far).  Returns the experts now resident."""
        if heat is not None:
            h = np.asarray(heat, dtype=np.float64)
            if h.shape != self.heat.shape:
                raise ValueError(f"heat profile has {h.shape[0]} entries, this layer has {self.n} experts")
            self.heat = h.copy()
        order = [int(e) for e in np.argsort(-self.heat, kind="stable")[: self.slots] if self.heat[e] > 0]
        if order:
            self._make_resident(order)
            self._unpin(order)
        return order

    # -- optimistic mode: device-only translation inside a captured step, misses settled afterwards ------------------
    def enable_optimistic(self, miss_count: torch.Tensor) -> None:
        """Steps may then be captured in a CUDA graph: :meth:`translate` never touches the host.  ``miss_count`` is one
        int32 device word shared by all layers of a model; the engine reads it once after a step."""
        self.optimistic = False  # the engine turns it on around a decode step; prefill and eager paths keep the waves
        self.miss_count = miss_count
        self.step_hist = torch.zeros(self.n, dtype=torch.int32, device=self.device)   # experts this step routed to
        self.heat_dev = torch.zeros(self.n, dtype=torch.int32, device=self.device)    # the same, accumulated
        self.stats.update({"replays": 0, "fallbacks": 0})

    def begin_step(self) -> None:
        self.step_hist.zero_()

    def translate(self, topk_ids: torch.Tensor) -> torch.Tensor:
        """Expert ids -> arena slots with what is resident NOW; routes to absent experts become -1 (the route plan skips
        them) and are counted.  Device work only: a gather, two scatter-adds, a sum."""
        valid = topk_ids >= 0
        ids = topk_ids.long().clamp(min=0)
        slot = self.slot_of_dev[ids]
        ones = valid.reshape(-1).to(torch.int32)
        self.step_hist.scatter_add_(0, ids.reshape(-1), ones)
        self.heat_dev.scatter_add_(0, ids.reshape(-1), ones)
        self.miss_count += (valid & (slot < 0)).sum().to(torch.int32)
        return torch.where(valid, slot, torch.full_like(slot, -1)).to(torch.int32)

    def settle(self) -> str:
        """After a step whose shared miss counter was not zero: make every expert THIS layer routed to resident.
        Returns ``"ok"`` (nothing was missing here), ``"replay"`` (uploads issued: run the step again) or
        ``"fallback"`` (the step needs more distinct experts than there are slots: run it in waves)."""
        hist = self.step_hist.cpu().numpy()
        used = [int(e) for e in np.flatnonzero(hist)]
        if all(self.slot_of[e] >= 0 for e in used):
            return "ok"
        if len(used) > self.slots:
            self.stats["fallbacks"] += 1
            return "fallback"
        self.heat = self.heat * self.decay + hist
        self._make_resident(used)
        self._unpin(used)  # pinned only while the set was being placed: nothing uploads during a replay
        self.stats["replays"] += 1
        return "replay"

    def absorb_heat(self) -> None:
        """Fold the device-side usage counts into the host heat (call between steps, before :meth:`rebalance`)."""
        if getattr(self, "heat_dev", None) is not None:
            self.heat = self.heat * self.decay + self.heat_dev.cpu().numpy()
            self.heat_dev.zero_()

    # -- between steps ------------------------------------------------------------------------------------------
    def rebalance(self, max_swaps: int = 4, hysteresis: float = 0.25) -> list[tuple[int, int]]:
        """Swap cold residents for hotter absent experts; returns the (evicted, loaded) pairs."""
        self.absorb_heat()
        swaps = native.moe_rank_swaps(self.heat, (self.slot_of >= 0).astype(np.uint8), max_swaps, hysteresis)
        done = []
        for evict, load in swaps:
            slot = int(self.slot_of[evict])
            if slot < 0 or self.book.pin(int(evict), 0) > 0:
                continue
            # re-key the slot: acquire for the newcomer evicts the LRU entry, so touch everything else first
            self.book.lookup(int(evict))
            for e in np.flatnonzero(self.slot_of >= 0):
                if e != evict:
                    self.book.lookup(int(e))
            got, evicted = self.book.acquire(int(load))
            if evicted is not None:
                self.slot_of[evicted] = -1
            self.slot_of[load] = got
            self._make_resident_noop_upload(int(load), got)
            done.append((int(evict), int(load)))
        self.slot_of_dev.copy_(torch.from_numpy(self.slot_of), non_blocking=True)
        return done

    def _make_resident_noop_upload(self, expert: int, slot: int) -> None:
        if self.copy_stream is not None:
            self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.copy_stream):
                self._upload(expert, slot)
            torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
        else:
            self._upload(expert, slot)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

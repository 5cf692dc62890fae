"""Session snapshots: the KV pages (and recurrent state) of a finished turn kept in host memory, so the next turn of
the same conversation restores them instead of prefilling the whole history again.

A snapshot belongs to a session id and records the token ids it covers; ``restore`` only applies it when those tokens
are a prefix of the new prompt (otherwise the conversation was edited and the snapshot is dropped).  Snapshots live
in an LRU bounded by bytes.  Unlike the content-addressed prefix cache this also works for models with recurrent
state (hybrid Gated-DeltaNet models), whose state cannot be cut at arbitrary block boundaries: the snapshot holds
the state exactly at its last token.  Reference: ``cpp_runtime/engine/include/session_snapshot_cache.h`` (in-RAM
per-session KV + recurrent snapshots).
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class Snapshot:
    tokens: list[int]
    pages: np.ndarray  # export of the pages that hold `tokens` (whole pages)
    recurrent: tuple[torch.Tensor, torch.Tensor] | None  # (conv, state) of the row, on the host
    nbytes: int


class SessionSnapshotCache:
    def __init__(self, budget_bytes: int = 8 << 30) -> None:
        self.budget = budget_bytes
        self.entries: OrderedDict[str, Snapshot] = OrderedDict()
        self.bytes = 0
        self.stats = {"saved": 0, "restored": 0, "dropped_mismatch": 0, "evicted": 0, "tokens_skipped": 0}

    def save(self, engine, row: int, session: str, tokens: list[int]) -> None:
        """Snapshot row ``row`` of ``engine`` as covering ``tokens`` (all of them must be in its KV pages)."""
        seq = engine.row_seq[row]
        ps = engine.cache.page_size
        n_pages = (len(tokens) + ps - 1) // ps
        pages = engine.cache.export_pages(engine.cache.allocator.owned[seq][:n_pages])
        rec = None
        if engine.rec_state is not None:
            rec = (engine.rec_state.conv[:, row].detach().cpu().clone(), engine.rec_state.state[:, row].detach().cpu().clone())
        nbytes = pages.nbytes + (sum(t.numel() * t.element_size() for t in rec) if rec else 0)
        self.drop(session)
        self.entries[session] = Snapshot(list(tokens), pages, rec, nbytes)
        self.bytes += nbytes
        self.stats["saved"] += 1
        while self.bytes > self.budget and len(self.entries) > 1:
            _, old = self.entries.popitem(last=False)
            self.bytes -= old.nbytes
            self.stats["evicted"] += 1

    def drop(self, session: str) -> None:
        old = self.entries.pop(session, None)
        if old is not None:
            self.bytes -= old.nbytes

    def restore(self, engine, row: int, session: str, prompt: list[int]) -> int:
        """Put the session's snapshot into row ``row`` (whose pages must already be assigned for ``prompt``) when it is
        a proper prefix of ``prompt``.  Returns the number of tokens restored (0: nothing usable)."""
        snap = self.entries.get(session)
        if snap is None:
            return 0
        n = len(snap.tokens)
        if n >= len(prompt) or list(prompt[:n]) != snap.tokens:
            self.drop(session)
            self.stats["dropped_mismatch"] += 1
            return 0
        self.entries.move_to_end(session)
        seq = engine.row_seq[row]
        ps = engine.cache.page_size
        n_pages = (n + ps - 1) // ps
        engine.cache.import_pages(engine.cache.allocator.owned[seq][:n_pages], snap.pages)
        if snap.recurrent is not None:
            engine.rec_state.conv[:, row].copy_(snap.recurrent[0])
            engine.rec_state.state[:, row].copy_(snap.recurrent[1])
        self.stats["restored"] += 1
        self.stats["tokens_skipped"] += n
        return n

"""Bookkeeping of the MTP draft/verify cycle (device kernels, with a plain-torch fallback for CPU tensors).

``prepare`` lays out the verify window ``[sampled, draft_0 .. draft_{K-1}]`` per row; ``accept`` keeps the longest
prefix of drafts that matches the verify arg-maxes, emits the confirmed tokens and advances the row state;
``select_rows`` picks the hidden state of the last confirmed position for chained drafts.
"""

from __future__ import annotations

import torch

from .lib import check, lib, ptr, stream_ptr


def prepare(sampled, draft, seq_lens, block_table, active, input_ids, positions, slots, window_lens, page_size: int) -> None:
    b, k = draft.shape
    w = k + 1
    if sampled.is_cuda:
        check(lib().mfq_mtp_prepare(ptr(sampled), ptr(draft), ptr(seq_lens), ptr(block_table), ptr(active), ptr(input_ids),
                                    ptr(positions), ptr(slots), ptr(window_lens), b, k, block_table.shape[1], page_size,
                                    stream_ptr()), "mtp_prepare")
        return
    on = active.bool() if active is not None else torch.ones(b, dtype=torch.bool)
    ids = torch.cat([sampled[:, None], draft], 1)
    pos = seq_lens[:, None] + torch.arange(w, dtype=torch.int32)[None]
    pages = block_table.gather(1, (pos // page_size).clamp(max=block_table.shape[1] - 1).long())
    sl = torch.where(on[:, None], pages * page_size + pos % page_size, torch.full_like(pos, -1))
    input_ids.copy_(ids.reshape(-1))
    positions.copy_(pos.reshape(-1))
    slots.copy_(sl.reshape(-1))
    window_lens.copy_(torch.where(on, seq_lens + w, seq_lens))


def accept(targets, head_next, active, draft, sampled, seq_lens, out_tokens, n_out, accept_row, stats) -> None:
    b, k = draft.shape
    w = k + 1
    if sampled.is_cuda:
        check(lib().mfq_mtp_accept(ptr(targets), ptr(head_next), ptr(active), ptr(draft), ptr(sampled), ptr(seq_lens),
                                   ptr(out_tokens), ptr(n_out), ptr(accept_row), ptr(stats), b, k, stream_ptr()), "mtp_accept")
        return
    tg, hn = targets.view(b, w), head_next.view(b, w)
    for r in range(b):
        if active is not None and not int(active[r]):
            n_out[r], accept_row[r] = 0, 0
            continue
        a = 0
        while a < k and int(draft[r, a]) == int(tg[r, a]):
            a += 1
        out_tokens[r] = -1
        out_tokens[r, : a + 1] = tg[r, : a + 1]
        n_out[r], accept_row[r] = a + 1, a
        sampled[r] = tg[r, a]
        seq_lens[r] += a + 1
        draft[r, 0] = hn[r, a]
        if stats is not None:
            stats[0] += k
            stats[1] += a


def select_rows(rows: torch.Tensor, accept_row: torch.Tensor, w: int, out: torch.Tensor | None = None) -> torch.Tensor:
    b = accept_row.numel()
    h = rows.shape[1]
    out = torch.empty((b, h), dtype=rows.dtype, device=rows.device) if out is None else out
    if rows.is_cuda:
        check(lib().mfq_mtp_select_rows(ptr(rows), ptr(accept_row), ptr(out), b, w, h, stream_ptr()), "mtp_select_rows")
    else:
        out.copy_(rows.view(b, w, h)[torch.arange(b), accept_row.long()])
    return out

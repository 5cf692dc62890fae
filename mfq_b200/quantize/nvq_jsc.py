"""NVQ-JSC quantizer: lattice codes whose group scale AND codebook bank come from one 4-bit state.

Plain NVQ gives every group of 24 weights a ``sub_bits``-wide multiple of the row anchor and one fixed codebook.  The
JSC variant (``formats/nvq.py: NvqJscTensor``) spends the same 4 bits on a STATE: ``scale_lut[state]`` is the group's
relative scale -- 16 free FP16 values instead of the integers 0..15 -- and ``bank_for_state[state]`` picks one of 1, 2 or
4 int8 magnitude tables, so a tensor can keep a fine table for small groups and a coarse one for large ones:

    w = anchor[row] * scale_lut[state] * codebooks[bank_for_state[state]][index] * sign

The encoder alternates, starting from the analytic tables (``analytic_jsc_tables``) and the base lattice in every bank:

1. assignment -- for every group the state, and for every vector the entry, with the least weighted error at the
   current anchors (per bank one pair of matrix products, then one pass per state);
2. anchors by least squares per row;
3. training (``train=True``): every ``scale_lut`` entry by least squares over the groups that chose it, every table
   entry as the scale-weighted mean of the vectors that chose it, rounded to int8 and kept non-negative; the state ->
   bank map stays ``state % banks``.  A round is kept only if it lowers the total error.

Signs are the even-parity coding of plain NVQ (``quantize/nvq.py: encode_even_parity``).
Reference: ``mfq/quantize/nvq_jsc.py`` (training loop, decode ``:1472-1500``), ``mfq/formats/nvq.py:425-520``.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..formats.nvq import NvqJscTensor, NvqSpec, analytic_jsc_tables, codebook as lattice
from .nvq import assign_fused, encode_even_parity, fused_assign_available

__all__ = ["quantize_nvq_jsc"]


def _assign_states(xv, wv, anchors_v, lut, bank_of, tables, vpg: int):
    """``xv, wv [V, vec]`` (V = groups * vpg, group-major), ``anchors_v [V]``.  Returns (state [G], index [G, vpg],
    error [G]) -- exhaustive over the 16 states, nearest entry per vector inside each."""
    v = xv.shape[0]
    g = v // vpg
    fused = fused_assign_available(xv, xv.shape[1])  # on a GPU: the fused nearest-codeword kernel, no [V, entries] matrices
    if not fused:
        cross = [(wv * xv) @ t.T for t in tables]
        quad = [wv @ (t * t).T for t in tables]
        x2 = (wv * xv * xv).sum(-1)
    best = torch.full((g,), float("inf"), device=xv.device)
    best_s = torch.zeros(g, dtype=torch.long, device=xv.device)
    best_i = torch.zeros((g, vpg), dtype=torch.long, device=xv.device)
    for s in range(16):
        b = int(bank_of[s])
        if fused:
            sc1 = (anchors_v * float(lut[s])).contiguous()
            idx = assign_fused(xv, wv, tables[b], sc1)
            diff = xv - sc1[:, None] * tables[b][idx]
            err = (wv * diff * diff).sum(-1).reshape(g, vpg).sum(-1)
        else:
            sc = (anchors_v * float(lut[s]))[:, None]
            val, idx = (sc * sc * quad[b] - 2.0 * sc * cross[b]).min(-1)
            err = (val + x2).reshape(g, vpg).sum(-1)
        take = err < best
        best = torch.where(take, err, best)
        best_s = torch.where(take, torch.full_like(best_s, s), best_s)
        best_i = torch.where(take[:, None], idx.reshape(g, vpg), best_i)
    return best_s, best_i, best


def quantize_nvq_jsc(weight, spec: NvqSpec | str = "e8_256", *, banks: int = 2, axis: int = 0, importance=None, train: bool = True,
                     learn_scales: bool = True, iterations: int = 4, storage_layout: str = "streams", device: str | torch.device = "cpu",
                     row_chunk: int = 128) -> NvqJscTensor:
    """``weight``: any-rank array whose ``axis`` indexes the rows.  ``spec``: a base grid name or an ``NvqSpec`` with
    group size 24, 4 sub bits and even-parity signs.  ``banks`` in (1, 2, 4).  ``train=False`` keeps the analytic state
    tables and the base lattice; ``learn_scales=False`` trains the banks but keeps the analytic scale table.
    ``storage_layout="group64"`` (4096-entry E8 grid only) packs one 64-bit record per group."""
    spec = NvqSpec(spec) if isinstance(spec, str) else spec
    if spec.groupsize != 24 or spec.sub_bits != 4 or spec.sign_mode != "even":
        raise ValueError("NVQ-JSC needs group size 24, 4-bit states and even-parity signs")
    if banks not in (1, 2, 4):
        raise ValueError("NVQ-JSC has 1, 2 or 4 codebook banks")
    w_full = torch.as_tensor(np.asarray(weight, dtype=np.float32))
    shape = tuple(w_full.shape)
    axis %= w_full.ndim
    rows_all = w_full.movedim(axis, 0).reshape(shape[axis], -1)
    out, n = rows_all.shape
    gs, vec = 24, spec.vector_size
    vpg = gs // vec
    ng = math.ceil(n / gs)
    padded = ng * gs
    nvec, nsign = math.ceil(n / vec), math.ceil(n / 8)
    dev = torch.device(device)
    rows = torch.nn.functional.pad(rows_all, (0, padded - n)).to(dev)
    wobj = torch.ones_like(rows) if importance is None else \
        torch.nn.functional.pad(torch.as_tensor(np.asarray(importance, dtype=np.float32)).reshape(1, n).expand(out, n), (0, padded - n)).to(dev).clone()
    wobj[:, n:] = 0.0
    target, masks = encode_even_parity(rows, torch.where(wobj > 0, wobj, torch.full_like(wobj, 1e-12)))
    lut_np, bank_np = analytic_jsc_tables(banks, vec)
    base = torch.as_tensor(lattice(spec).astype(np.float32), device=dev)
    tables = [base.clone() for _ in range(banks)]
    lut = torch.as_tensor(lut_np.astype(np.float32), device=dev)
    top_code = float(base.max()) * float(lut.max())
    anchors = (target.abs().amax(1) / max(top_code, 1e-12)).clamp_min(1e-12).half().float()

    def assign_all(anchors, lut, tables):
        st = torch.zeros((out, ng), dtype=torch.long, device=dev)
        ix = torch.zeros((out, ng, vpg), dtype=torch.long, device=dev)
        er = torch.zeros((out, ng), device=dev)
        for r0 in range(0, out, row_chunk):
            r1 = min(out, r0 + row_chunk)
            xv = target[r0:r1].reshape(-1, vec)
            wv = wobj[r0:r1].reshape(-1, vec)
            av = anchors[r0:r1].repeat_interleave(ng * vpg)
            s, i, e = _assign_states(xv, wv, av, lut, bank_np, tables, vpg)
            st[r0:r1], ix[r0:r1], er[r0:r1] = s.reshape(-1, ng), i.reshape(-1, ng, vpg), e.reshape(-1, ng)
        return st, ix, er

    def codes_of(st, ix, tables):
        bank = torch.as_tensor(bank_np.astype(np.int64), device=dev)[st]                      # [out, ng]
        stack = torch.stack(tables)                                                           # [banks, entries, vec]
        return stack[bank[:, :, None].expand(-1, -1, vpg), ix].reshape(out, ng, gs)           # magnitudes per weight

    def refit_anchors(st, ix, lut, tables, anchors):
        code = codes_of(st, ix, tables) * lut[st][:, :, None]
        tg, wg = target.reshape(out, ng, gs), wobj.reshape(out, ng, gs)
        num, den = (wg * tg * code).sum((1, 2)), (wg * code * code).sum((1, 2))
        a = torch.where(den > 0, num / den.clamp_min(1e-30), anchors).clamp(0, 65504.0)
        return a.half().float()

    st, ix, er = assign_all(anchors, lut, tables)
    anchors = refit_anchors(st, ix, lut, tables, anchors)
    st, ix, er = assign_all(anchors, lut, tables)
    best = (float(er.sum()), anchors, lut, [t.clone() for t in tables], st, ix)
    if train:
        tg, wg = target.reshape(out, ng, gs), wobj.reshape(out, ng, gs)
        bank_t = torch.as_tensor(bank_np.astype(np.int64), device=dev)
        for _ in range(max(1, iterations)):
            # state scales: least squares over the groups of each state
            code = codes_of(st, ix, tables) * anchors[:, None, None]
            num = torch.zeros(16, device=dev).index_add_(0, st.reshape(-1), (wg * tg * code).sum(-1).reshape(-1))
            den = torch.zeros(16, device=dev).index_add_(0, st.reshape(-1), (wg * code * code).sum(-1).reshape(-1))
            if learn_scales:
                lut = torch.where(den > 0, num / den.clamp_min(1e-30), lut).clamp(0, 65504.0).half().float()
            # table entries: scale-weighted mean of their vectors, in code units
            sc = (anchors[:, None] * lut[st])[:, :, None].expand(-1, -1, vpg).reshape(-1)                     # [V]
            xv, wv = target.reshape(-1, vec), wobj.reshape(-1, vec)
            bank_v = bank_t[st][:, :, None].expand(-1, -1, vpg).reshape(-1)
            flat = bank_v * spec.entries + ix.reshape(-1)
            num_e = torch.zeros((banks * spec.entries, vec), device=dev).index_add_(0, flat, wv * xv * sc[:, None])
            den_e = torch.zeros((banks * spec.entries, vec), device=dev).index_add_(0, flat, wv * (sc * sc)[:, None])
            old = torch.stack(tables).reshape(-1, vec)
            new = torch.where(den_e > 0, num_e / den_e.clamp_min(1e-30), old).round().clamp(0, 127)
            tables = list(new.reshape(banks, spec.entries, vec))
            st, ix, er = assign_all(anchors, lut, tables)
            anchors = refit_anchors(st, ix, lut, tables, anchors)
            st, ix, er = assign_all(anchors, lut, tables)
            total = float(er.sum())
            if total < best[0]:
                best = (total, anchors, lut, [t.clone() for t in tables], st, ix)
    _total, anchors, lut, tables, st, ix = best
    idx_dtype = np.uint16 if spec.index_bits > 8 else np.uint8
    return NvqJscTensor(
        base_spec=spec, shape=shape, axis=axis, neuron_len=n, neuron_scale=anchors.cpu().numpy().astype(np.float32),
        scale_lut=lut.cpu().numpy().astype(np.float32), bank_for_state=bank_np.astype(np.uint8),
        codebooks=torch.stack(tables).round().to(torch.int8).cpu().numpy(), state=st.cpu().numpy().astype(np.uint8),
        indices=ix.reshape(out, ng * vpg)[:, :nvec].cpu().numpy().astype(idx_dtype),
        signs=masks[:, :nsign].cpu().numpy().astype(np.uint8), storage_layout=storage_layout)

"""NINT quantizer: per-group weighted least-squares affine fit, then row anchoring.

Algorithm (same steps as the reference NumPy quantizer, ``mfq/formats/nint.py:364-475``,
itself the k-quant ``make_qkx2`` search of llama.cpp), restated batched over
``[rows, groups, gs]`` in torch so that it runs on CPU or on the GPU:

1. group weights ``w = rms(group) + |x|`` (or an importance vector), zero on K padding;
2. for the plain min/max grid and ``nstep+1`` perturbed inverse scales, round to
   levels ``L`` and solve the 2x2 weighted normal equations for ``(scale, min)``
   with ``min <= 0``; keep the candidate with the lowest weighted error;
3. anchors ``d = f16(max_g scale / (2^k-1))``, ``dmin = f16(max_g -min / (2^k-1))``;
   group codes ``rint((2^k-1) * scale / max scale)``;
4. re-round element codes against the *effective* (anchored) scale and min.

With an importance vector (an imatrix) the search is the weighted variant (reference:
``mfq/quantize/nint_quant.py:102-139,141-217,310-480``): element weights ``imp * sqrt(sigma2 + x^2)`` with ``sigma2``
taken over 256-value blocks, a finer candidate grid (37 inverse scales from ``qmax - 0.9`` in steps of 0.05), and a
final coordinate descent on what is actually stored -- the integer group codes are re-solved against the anchored row
scale / minimum and the element codes re-rounded, a step being kept only when the weighted error of the stored
reconstruction falls.
"""

from __future__ import annotations

import numpy as np
import torch

from ..formats.nint import NintSpec, NintTensor

__all__ = ["quantize_nint", "fit_groups", "importance_weights", "refine_stored"]


def fit_groups(x: torch.Tensor, w: torch.Tensor, qmax: int, fine: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Best ``(scale, zero)`` per group with ``recon = zero + scale * L``, ``L in [0, qmax]``.

    ``x``/``w`` are ``[..., gs]``; returns two ``[...]`` tensors (``zero <= 0``).  ``fine``: the denser candidate grid of
    the importance-weighted search.
    """
    if fine:
        rmin, rdelta, nstep = -0.9, 0.05, 36
    else:
        rmin, rdelta, nstep = (-1.0, 0.1, 20) if qmax <= 15 else (-0.5, 0.1, 15)
    lo = torch.clamp(x.amin(-1), max=0.0)
    hi = x.amax(-1)
    sw = w.sum(-1)
    sx = (w * x).sum(-1)
    flat = (hi == lo) | (sw <= 0)
    span = torch.where(flat, torch.ones_like(hi), hi - lo)
    shifted = x - lo[..., None]

    inv = qmax / span
    lv = torch.clamp(torch.round(inv[..., None] * shifted), 0, qmax)
    err0 = lv / inv[..., None] + lo[..., None] - x
    best_err = (w * err0 * err0).sum(-1)
    best_scale = 1.0 / inv
    best_zero = lo.clone()
    for step in range(nstep + 1):
        inv = (rmin + rdelta * step + qmax) / span
        lv = torch.clamp(torch.round(inv[..., None] * shifted), 0, qmax)
        sl = (w * lv).sum(-1)
        sl2 = (w * lv * lv).sum(-1)
        sxl = (w * lv * x).sum(-1)
        det = sw * sl2 - sl * sl
        ok = det > 0
        den = torch.where(ok, det, torch.ones_like(det))
        sc = (sw * sxl - sx * sl) / den
        zp = (sl2 * sx - sl * sxl) / den
        over = zp > 0  # zero point must stay <= 0: refit a pure scale
        sc = torch.where(over, sxl / torch.where(sl2 > 0, sl2, torch.ones_like(sl2)), sc)
        zp = torch.where(over, torch.zeros_like(zp), zp)
        diff = sc[..., None] * lv + zp[..., None] - x
        err = (w * diff * diff).sum(-1)
        take = ok & (err < best_err)
        best_err = torch.where(take, err, best_err)
        best_scale = torch.where(take, sc, best_scale)
        best_zero = torch.where(take, zp, best_zero)
    best_scale = torch.where(flat, torch.zeros_like(best_scale), best_scale)
    best_zero = torch.where(flat, lo, best_zero)
    return best_scale, best_zero


def _f16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).to(torch.float32)


IMATRIX_BLOCK = 256  # sigma^2 of the importance weights is taken over blocks of this many inputs


def importance_weights(rows: torch.Tensor, importance: torch.Tensor) -> torch.Tensor:
    """Element weights of the importance-weighted search: ``imp[k] * sqrt(sigma2[block(k)] + x^2)`` with
    ``sigma2 = 2 * mean(x^2)`` over blocks of 256 inputs (the last block over what it holds)."""
    out, n = rows.shape
    pad = (-n) % IMATRIX_BLOCK
    blocks = torch.nn.functional.pad(rows, (0, pad)).reshape(out, -1, IMATRIX_BLOCK)
    counts = torch.full((blocks.shape[1],), float(IMATRIX_BLOCK), device=rows.device)
    if pad:
        counts[-1] -= pad
    sigma2 = 2.0 * blocks.pow(2).sum(-1) / counts[None, :]
    sigma2 = sigma2.repeat_interleave(IMATRIX_BLOCK, dim=1)[:, :n]
    return importance.expand(out, n) * torch.sqrt(sigma2 + rows * rows)


def refine_stored(x, w, q, d, dm, ls, lm, qmax: int, kmax: int, passes: int = 2):
    """Coordinate descent on the stored reconstruction ``d * ls * q - dm * lm`` (weighted squared error): with the element
    codes fixed each group's best integer ``ls`` and ``lm`` have closed forms; then the element codes are re-rounded
    against the new effective values.  A pass is kept per row only where the row's weighted error fell."""
    def row_error(q_, ls_, lm_):
        rec = (d[:, None] * ls_)[..., None] * q_ - (dm[:, None] * lm_)[..., None]
        return (w * (rec - x) ** 2).sum((-1, -2))
    best = row_error(q, ls, lm)
    for _ in range(passes):
        cls, clm, cq = ls.clone(), lm.clone(), q.clone()
        for _inner in range(2):
            sw, sx = w.sum(-1), (w * x).sum(-1)
            sq, sq2, sqx = (w * cq).sum(-1), (w * cq * cq).sum(-1), (w * cq * x).sum(-1)
            em = dm[:, None] * clm
            den = d[:, None] * sq2
            new_ls = torch.where(den > 0, torch.clamp(torch.round((sqx + em * sq) / den.clamp_min(1e-30)), 0, kmax), cls)
            es = d[:, None] * new_ls
            den_m = dm[:, None] * sw
            new_lm = torch.where(den_m > 0, torch.clamp(torch.round((es * sq - sx) / den_m.clamp_min(1e-30)), 0, kmax), clm)
            cls, clm = new_ls, new_lm
        es, em = d[:, None] * cls, dm[:, None] * clm
        cq = torch.clamp(torch.round((x + em[..., None]) / torch.where(es > 0, es, torch.ones_like(es))[..., None]), 0, qmax)
        err = row_error(cq, cls, clm)
        better = err < best
        if not bool(better.any()):
            break
        q = torch.where(better[:, None, None], cq, q)
        ls = torch.where(better[:, None], cls, ls)
        lm = torch.where(better[:, None], clm, lm)
        best = torch.where(better, err, best)
    return q, ls, lm


def _quantize_uniform(rows: torch.Tensor, bits: int, gs: int, k: int, importance: torch.Tensor | None):
    out, n = rows.shape
    pad = (-n) % gs
    x = torch.nn.functional.pad(rows, (0, pad)).reshape(out, -1, gs)
    if importance is None:
        w = x.pow(2).mean(-1, keepdim=True).sqrt() + x.abs()
    else:
        w = torch.nn.functional.pad(importance_weights(rows, importance), (0, pad)).reshape(out, -1, gs).clone()
    if pad:
        w[:, -1, gs - pad:] = 0.0
    qmax, kmax = (1 << bits) - 1, (1 << k) - 1
    scale, zero = fit_groups(x, w, qmax, fine=importance is not None)
    mins = -zero
    top_s = scale.amax(-1)
    top_m = mins.amax(-1)
    d = torch.where(top_s > 0, _f16(top_s / kmax), torch.zeros_like(top_s))
    dm = torch.where(top_m > 0, _f16(top_m / kmax), torch.zeros_like(top_m))
    ls = torch.where(top_s[:, None] > 0, torch.clamp(torch.round(kmax * scale / top_s.clamp_min(1e-30)[:, None]), 0, kmax), torch.zeros_like(scale))
    lm = torch.where(top_m[:, None] > 0, torch.clamp(torch.round(kmax * mins / top_m.clamp_min(1e-30)[:, None]), 0, kmax), torch.zeros_like(mins))
    eff_s = d[:, None] * ls
    eff_m = dm[:, None] * lm
    q = torch.clamp(torch.round((x + eff_m[..., None]) / torch.where(eff_s > 0, eff_s, torch.ones_like(eff_s))[..., None]), 0, qmax)
    if importance is not None:
        q, ls, lm = refine_stored(x, w, q, d, dm, ls, lm, qmax, kmax)
    return q.to(torch.uint8), d, dm, ls.to(torch.uint8), lm.to(torch.uint8)


def quantize_nint(weight, spec: NintSpec = NintSpec(), *, axis: int = 0, row_q_bits=None, row_sub_bits=None,
                  importance=None, device: str | torch.device = "cpu", row_chunk: int = 4096) -> NintTensor:
    """Quantize ``weight`` (any rank >= 2; ``axis`` indexes output neurons) to NINT.

    ``row_q_bits`` / ``row_sub_bits`` give per-neuron widths (NINTv2 allocation);
    ``importance`` is an optional non-negative weight per input coordinate.
    """
    w = torch.as_tensor(np.asarray(weight, dtype=np.float32) if not torch.is_tensor(weight) else weight).to(torch.float32)
    shape = tuple(w.shape)
    axis %= w.ndim
    rows = w.movedim(axis, 0).reshape(shape[axis], -1).to(device)
    out, n = rows.shape
    gs = spec.groupsize
    ng = (n + gs - 1) // gs
    qw = np.full(out, spec.bits, dtype=np.uint8) if row_q_bits is None else np.asarray(row_q_bits, dtype=np.uint8)
    kw = np.full(out, spec.sub_bits, dtype=np.uint8) if row_sub_bits is None else np.asarray(row_sub_bits, dtype=np.uint8)
    imp = None if importance is None else torch.as_tensor(np.asarray(importance, dtype=np.float32)).reshape(1, n).to(device)
    q = np.zeros((out, ng, gs), dtype=np.uint8)
    d = np.zeros(out, dtype=np.float32)
    dm = np.zeros(out, dtype=np.float32)
    ls = np.zeros((out, ng), dtype=np.uint8)
    lm = np.zeros((out, ng), dtype=np.uint8)
    for bits, k in sorted({(int(a), int(b)) for a, b in zip(qw, kw)}):
        sel = np.flatnonzero((qw == bits) & (kw == k))
        for start in range(0, sel.size, row_chunk):
            idx = sel[start : start + row_chunk]
            tq, td, tdm, tls, tlm = _quantize_uniform(rows[torch.as_tensor(idx, device=rows.device)], bits, gs, k, imp)
            q[idx], d[idx], dm[idx] = tq.cpu().numpy(), td.cpu().numpy(), tdm.cpu().numpy()
            ls[idx], lm[idx] = tls.cpu().numpy(), tlm.cpu().numpy()
    return NintTensor(
        spec=spec, shape=shape, axis=axis, neuron_len=n, q=q, neuron_scale=d, neuron_min=dm, sub_scale=ls, sub_min=lm,
        row_q_bits=None if row_q_bits is None else qw, row_sub_bits=None if row_sub_bits is None else kw,
    )

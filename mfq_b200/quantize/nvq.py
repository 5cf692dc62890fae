"""NVQ quantizer: even-parity sign coding + joint lattice-index / group-scale search.

Steps (same pipeline as the reference, ``mfq/quantize/nvq_quant.py:170-240,453-600``),
restated as batched torch so the nearest-codeword search is two GEMMs per chunk:

1. signs: 7 free sign bits per 8 weights, the 8th is their parity.  A block whose
   true signs have odd parity gives up the sign of its cheapest element
   (smallest ``w*x^2``); the magnitude target of that element becomes ``-|x|``.
2. per group, ``search_steps`` trial scales ``max|x| / (qmax + offset)``; for each:
   nearest codeword per vector under the weighted metric
   ``argmin_c  s^2 * (w . c^2) - 2 s * ((w*x) . c)``, weighted-LS refit of the
   scale, one more assignment + refit; keep the lowest error.
3. row anchor ``d = f16(max_g scale / (2^k-1))``, group codes ``rint(scale / d)``;
   re-assign at the effective scales, refit the anchor in closed form, repeat once.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..formats.nvq import NvqSpec, NvqTensor, codebook as lattice

__all__ = ["quantize_nvq", "encode_even_parity", "train_tensor_codebook"]


def encode_even_parity(rows: torch.Tensor, w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Return (magnitude targets ``[out, K8]``, 7-bit sign masks ``[out, K8/8]``)."""
    out, n = rows.shape
    blk = rows.reshape(out, n // 8, 8)
    neg = blk < 0
    odd = (neg.sum(-1) & 1).bool()
    cost = (w.reshape(out, n // 8, 8) * blk * blk)
    victim = cost.argmin(-1)
    flip = torch.zeros_like(neg)
    flip.scatter_(-1, victim[..., None], odd[..., None])
    stored = neg ^ flip
    target = torch.where(flip, -blk.abs(), blk.abs())
    bitw = (1 << torch.arange(7, device=rows.device)).to(torch.int32)
    masks = (stored[..., :7].to(torch.int32) * bitw).sum(-1).to(torch.uint8)
    return target.reshape(out, n), masks


def _assign(cross: torch.Tensor, quad: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    s = scale[:, None]
    return (s * s * quad - 2.0 * s * cross).argmin(-1)


def fused_assign_available(x: torch.Tensor, vec: int) -> bool:
    """The fused CUDA assignment (``ops/csrc/quant_ops.cu``) serves CUDA tensors with 4- or 8-wide vectors."""
    if not x.is_cuda or vec not in (4, 8):
        return False
    from ..ops import lib as _lib
    return _lib.available()


def assign_fused(xv: torch.Tensor, wv: torch.Tensor, table: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Nearest codeword of every vector under the weighted error, without the ``[V, C]`` cost matrices:
    ``xv, wv [V, vec]``, ``table [C, vec]``, ``scale [V]`` -> indices ``[V]`` (int64)."""
    from ..ops.lib import check, lib, ptr, stream_ptr
    v, vec = xv.shape
    idx = torch.empty(v, dtype=torch.int32, device=xv.device)
    rc = lib().mfq_nvq_assign(ptr(xv.contiguous()), ptr(wv.contiguous()), ptr(scale.contiguous().float()),
                              ptr(table.contiguous().float()), ptr(idx), v, table.shape[0], vec, stream_ptr())
    check(rc, "nvq_assign")
    return idx.to(torch.int64)


def _refit(xg, wg, idx, table, vpg):
    code = table[idx].reshape(xg.shape)
    num = (wg * xg * code).sum(-1)
    den = (wg * code * code).sum(-1)
    return torch.where(den > 0, num / den.clamp_min(1e-30), torch.zeros_like(num)).clamp_min(0.0), code


def _search(xg: torch.Tensor, wg: torch.Tensor, table: torch.Tensor, vec: int, steps: int):
    g, gs = xg.shape
    vpg = gs // vec
    xv = xg.reshape(g * vpg, vec)
    wv = wg.reshape(g * vpg, vec)
    fused = fused_assign_available(xg, vec)
    if fused:
        cross = quad = None  # never materialised on the GPU path
        assign = lambda sc: assign_fused(xv, wv, table, sc)
    else:
        cross = (wv * xv) @ table.T
        quad = wv @ (table * table).T
        assign = lambda sc: _assign(cross, quad, sc)
    qmax = float(table.max())
    amax = xg.abs().amax(-1)
    best_err = torch.full((g,), float("inf"), device=xg.device)
    best_scale = torch.zeros(g, device=xg.device)
    best_idx = torch.zeros((g, vpg), dtype=torch.long, device=xg.device)
    for off in torch.linspace(-0.12 * qmax, 0.12 * qmax, steps).tolist():
        s0 = torch.where(amax > 0, amax / (qmax + off), torch.zeros_like(amax))
        idx = assign(s0.repeat_interleave(vpg)).reshape(g, vpg)
        s1, _ = _refit(xg, wg, idx, table, vpg)
        idx = assign(s1.repeat_interleave(vpg)).reshape(g, vpg)
        s2, code = _refit(xg, wg, idx, table, vpg)
        diff = s2[:, None] * code - xg
        err = (wg * diff * diff).sum(-1)
        take = err < best_err
        best_err = torch.where(take, err, best_err)
        best_scale = torch.where(take, s2, best_scale)
        best_idx[take] = idx[take]
    return best_scale, best_idx, assign


def train_tensor_codebook(weight, spec: NvqSpec, *, axis: int = 0, importance=None, rounds: int = 3, sample_rows: int = 2048,
                          search_steps: int = 7, seed: int = 0, device: str | torch.device = "cpu") -> np.ndarray:
    """A codebook of ``spec.entries`` magnitude vectors fitted to ONE tensor (stored in its blob, 2 bytes per entry).
    Entries stay on the format's alphabet -- odd integers up to 7 (8-wide) or 15 (4-wide).  Lloyd rounds from the
    standard grid on at most ``sample_rows`` rows: assign with the joint index / scale search, move every coordinate of
    every entry to the odd level with the least weighted error over its vectors, and give entries that ended up unused
    or duplicated the most frequent rounded target vectors the book does not hold yet.
    Reference: ``mfq/quantize/nvq_tensor_codebook.py`` (tensor-local codebooks), ``nvq_codebook.py`` (alphabet rules)."""
    w_full = torch.as_tensor(np.asarray(weight, dtype=np.float32))
    axis %= w_full.ndim
    rows_all = w_full.movedim(axis, 0).reshape(w_full.shape[axis], -1)
    out, n = rows_all.shape
    gs, vec = spec.groupsize, spec.vector_size
    ng = math.ceil(n / gs)
    g = torch.Generator().manual_seed(seed)
    pick = torch.randperm(out, generator=g)[:sample_rows].sort().values
    rows = torch.nn.functional.pad(rows_all[pick], (0, ng * gs - n)).to(device)
    o = rows.shape[0]
    wobj = torch.ones_like(rows) if importance is None else \
        torch.nn.functional.pad(torch.as_tensor(np.asarray(importance, dtype=np.float32)).reshape(1, n).expand(o, n), (0, ng * gs - n)).to(device).clone()
    wobj[:, n:] = 0.0
    target, _ = encode_even_parity(rows, torch.where(wobj > 0, wobj, torch.full_like(wobj, 1e-12)))
    xg, wg = target.reshape(o * ng, gs), wobj.reshape(o * ng, gs)
    vpg = gs // vec
    top = 7 if vec == 8 else 15
    levels = torch.arange(1, top + 1, 2, dtype=torch.float32, device=rows.device)
    table = torch.as_tensor(lattice(spec).astype(np.float32), device=rows.device)

    def total_error(tab):
        scale, idx, _ = _search(xg, wg, tab, vec, search_steps)
        diff = scale[:, None] * tab[idx].reshape(xg.shape) - xg
        return float((wg * diff * diff).sum()), scale, idx

    best_err, scale, idx = total_error(table)
    best = table.clone()
    for _ in range(max(1, rounds)):
        sv = scale.repeat_interleave(vpg)                                     # [V]
        xv, wv, iv = xg.reshape(-1, vec), wg.reshape(-1, vec), idx.reshape(-1)
        live = sv > 0
        xv, wv, iv, sv = xv[live], wv[live], iv[live], sv[live]
        cost = torch.zeros((spec.entries, vec, levels.numel()), device=rows.device)
        for li, level in enumerate(levels):
            cost[:, :, li].index_add_(0, iv, wv * (xv - sv[:, None] * level) ** 2)
        used = torch.zeros(spec.entries, dtype=torch.bool, device=rows.device)
        used[iv.unique()] = True
        new = table.clone()
        new[used] = levels[cost[used].argmin(-1)]
        # unused and duplicate slots: the most frequent rounded targets that are not in the book yet
        snapped = levels[((xv / sv[:, None]).clamp(1, top)[..., None] - levels).abs().argmin(-1)]
        uniq, counts = torch.unique(snapped, dim=0, return_counts=True)
        order = counts.argsort(descending=True)
        held, free = set(), []
        rows_np = new.cpu().numpy().astype(np.int8)
        for e in range(spec.entries):
            key = rows_np[e].tobytes()
            if key in held or not bool(used[e]):
                free.append(e)
            else:
                held.add(key)
        cand = uniq[order].cpu().numpy().astype(np.int8)
        c = 0
        spare = lattice(spec).astype(np.int8)
        for e in free:
            while c < cand.shape[0] and cand[c].tobytes() in held:
                c += 1
            if c < cand.shape[0]:
                rows_np[e] = cand[c]
            else:  # nothing left to add from the data: keep a grid entry that is not held (a book may not repeat itself)
                rows_np[e] = next(sp for sp in spare if sp.tobytes() not in held)
            held.add(rows_np[e].tobytes())
        table = torch.as_tensor(rows_np.astype(np.float32), device=rows.device)
        err, scale, idx = total_error(table)
        if err < best_err:
            best_err, best = err, table.clone()
    return best.cpu().numpy().astype(np.int8)


def quantize_nvq(weight, spec: NvqSpec, *, axis: int = 0, importance=None, search_steps: int = 19,
                 refit_anchor: bool = True, device: str | torch.device = "cpu", row_chunk: int = 256,
                 codebook: np.ndarray | None = None) -> NvqTensor:
    """``codebook``: a tensor-local table (``train_tensor_codebook``) carried in the blob instead of the standard grid."""
    if spec.sign_mode != "even":
        raise NotImplementedError("the quantizer emits even-parity signs only")
    w_full = torch.as_tensor(np.asarray(weight, dtype=np.float32) if not torch.is_tensor(weight) else weight).to(torch.float32)
    shape = tuple(w_full.shape)
    axis %= w_full.ndim
    rows_all = w_full.movedim(axis, 0).reshape(shape[axis], -1)
    out, n = rows_all.shape
    gs, vec = spec.groupsize, spec.vector_size
    ng = math.ceil(n / gs)
    padded = ng * gs
    table = torch.as_tensor((lattice(spec) if codebook is None else np.asarray(codebook)).astype(np.float32), device=device)
    levels = (1 << spec.sub_bits) - 1
    nvec, nsign = math.ceil(n / vec), math.ceil(n / 8)
    d_all = np.zeros(out, np.float32)
    s_all = np.zeros((out, ng), np.uint8)
    i_all = np.zeros((out, nvec), np.uint16 if spec.index_bits > 8 else np.uint8)
    m_all = np.zeros((out, nsign), np.uint8)
    imp = None if importance is None else torch.as_tensor(np.asarray(importance, dtype=np.float32)).reshape(1, n)
    for r0 in range(0, out, row_chunk):
        rows = torch.nn.functional.pad(rows_all[r0 : r0 + row_chunk], (0, padded - n)).to(device)
        o = rows.shape[0]
        wobj = torch.ones_like(rows) if imp is None else torch.nn.functional.pad(imp.expand(o, n), (0, padded - n)).to(device).clone()
        if padded > n:
            wobj[:, n:] = 0.0
        target, masks = encode_even_parity(rows, torch.where(wobj > 0, wobj, torch.full_like(wobj, 1e-12)))
        xg = target.reshape(o * ng, gs)
        wg = wobj.reshape(o * ng, gs)
        raw, idx, assign = _search(xg, wg, table, vec, search_steps)
        raw2 = raw.reshape(o, ng)
        top = raw2.amax(-1)
        d = torch.where(top > 0, (top / levels).to(torch.float16).to(torch.float32), torch.zeros_like(top))
        sub = torch.clamp(torch.round(raw2 / torch.where(d > 0, d, torch.ones_like(d))[:, None]), 0, levels)
        vpg = gs // vec

        def reassign(anchor):
            eff = (anchor[:, None] * sub).reshape(-1)
            return assign(eff.repeat_interleave(vpg)).reshape(o * ng, vpg)

        def refit(index):
            code = table[index].reshape(o, ng, gs) * sub[:, :, None]
            num = (wg.reshape(o, ng, gs) * xg.reshape(o, ng, gs) * code).sum((-1, -2))
            den = (wg.reshape(o, ng, gs) * code * code).sum((-1, -2))
            a = torch.where(den > 0, num / den.clamp_min(1e-30), torch.zeros_like(num)).clamp_min(0.0)
            return a.to(torch.float16).to(torch.float32)

        idx = reassign(d)
        if refit_anchor:
            d = refit(idx)
            idx = reassign(d)
            d = refit(idx)
        sl = slice(r0, r0 + o)
        d_all[sl] = d.cpu().numpy()
        s_all[sl] = sub.to(torch.uint8).cpu().numpy()
        i_all[sl] = idx.reshape(o, ng * vpg)[:, :nvec].cpu().numpy().astype(i_all.dtype)
        m_all[sl] = masks[:, :nsign].cpu().numpy()
    return NvqTensor(spec=spec, shape=shape, axis=axis, neuron_len=n, neuron_scale=d_all, sub_scale=s_all,
                     indices=i_all, signs=m_all, codebook=None if codebook is None else np.asarray(codebook, dtype=np.int8))

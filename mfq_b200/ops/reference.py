"""Plain PyTorch (fp32) restatements of every fused kernel: the numerical oracle of the GPU tests and the
CPU execution path of the models."""

from __future__ import annotations

import math

import torch

E4M3_MAX = 448.0
FP8 = torch.float8_e4m3fn


def quant_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    scale = xf.abs().amax(-1).clamp_min(1e-12) / E4M3_MAX
    q = (xf / scale[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(FP8)
    return q, scale


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(torch.bfloat16)


def rmsnorm_quant(x, w, eps, residual=None):
    if residual is not None:
        x = (x.float() + residual.float()).to(torch.bfloat16)
    y = rmsnorm(x, w, eps)
    q, s = quant_rows(y)
    return q, s, y, x


def silu_mul_quant(gate_up: torch.Tensor):
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    h = (g / (1 + torch.exp(-g)) * u).to(torch.bfloat16)
    return quant_rows(h)


def dequant_block(w_q: torch.Tensor, w_scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    n, k = w_q.shape
    s = w_scale.repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return w_q.float() * s


def fp8_gemm(x_q, x_scale, w_q, w_scale, residual=None) -> torch.Tensor:
    y = (x_q.float() * x_scale[:, None]) @ dequant_block(w_q, w_scale).T
    if residual is not None:
        y = y + residual.float()
    return y.to(torch.bfloat16)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, rot: int | None = None, scaling=None) -> torch.Tensor:
    """``x [T, H, D]``; rotate-half pairing (i, i + rot/2) over the first ``rot`` dims.  ``scaling``: a
    :class:`~mfq_b200.models.rope_scaling.YarnScaling` (blended frequencies, cos / sin times its attention factor)."""
    d = x.shape[-1]
    rot = rot or d
    half = rot // 2
    if scaling is not None:
        inv, mscale = scaling.inv_freq(rot, theta, x.device), scaling.mscale
    else:
        inv, mscale = torch.exp2(-math.log2(theta) * (2 * torch.arange(half, device=x.device, dtype=torch.float32)) / rot), 1.0
    ang = positions.float()[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :] * mscale, ang.sin()[:, None, :] * mscale
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = xf.clone()
    out[..., :half] = a * c - b * s
    out[..., half:rot] = b * c + a * s
    return out.to(torch.bfloat16)


def quant_kv(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[T, H, D]`` bf16 -> fp8 codes + one multiplier per (token, head)."""
    xf = x.float()
    scale = xf.abs().amax(-1).clamp_min(1e-12) / E4M3_MAX
    return (xf / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(FP8), scale


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: float, causal_offset: int | None = None):
    """``q [Tq, Hq, D]``, ``k/v [Tk, Hk, D]`` (float).  Query i sees keys ``<= i + causal_offset``."""
    tq, hq, d = q.shape
    tk, hk, _ = k.shape
    g = hq // hk
    kf = k.float().repeat_interleave(g, 1)
    vf = v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * sm_scale
    if causal_offset is not None:
        qi = torch.arange(tq, device=q.device)[:, None] + causal_offset
        ki = torch.arange(tk, device=q.device)[None, :]
        s = s.masked_fill((ki > qi)[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vf).to(torch.bfloat16)


def gather_paged(kv, block_table_row: torch.Tensor, length: int):
    """Dequantized ``k, v [length, Hk, D]`` of one sequence from a :class:`LayerKV` (physical page layout)."""
    pos = torch.arange(length, device=kv.k.device)
    return gather_slots(kv, block_table_row.long()[pos // kv.page_size] * kv.page_size + pos % kv.page_size)


def gather_slots(kv, slots: torch.Tensor):
    """Dequantized ``k, v [T, Hk, D]`` rows at physical slots (page * page_size + offset)."""
    from ..engine.kv_cache import V_SLOT_OF_TOKEN
    ps = kv.page_size
    pages, off = (slots // ps).long(), (slots % ps).long()
    k = kv.k[pages, :, :, off]  # [T, Hk, D/64, 64]
    k = k.reshape(k.shape[0], k.shape[1], -1).float() * kv.k_scale[pages, :, off][..., None]
    vslot = torch.tensor(V_SLOT_OF_TOKEN, device=slots.device)[off]
    v = kv.v[pages, :, :, vslot].float() * kv.v_scale[pages, :, off][..., None]
    return k, v


def paged_attn_decode(q, kv, block_table, seq_lens, sm_scale, q_len: int = 1):
    outs = []
    b = q.shape[0] // q_len
    for i in range(b):
        n = int(seq_lens[i])
        if n <= 0:  # an unused row of the batch bucket: nothing to attend to (the GPU kernel writes zeros too)
            outs.append(torch.zeros_like(q[i * q_len : (i + 1) * q_len]))
            continue
        k, v = gather_paged(kv, block_table[i], n)
        outs.append(attention(q[i * q_len : (i + 1) * q_len], k, v, sm_scale, causal_offset=n - q_len))
    return torch.cat(outs, 0)


def write_kv(kv, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor) -> None:
    from ..engine.kv_cache import V_SLOT_OF_TOKEN
    kq, ks = quant_kv(k)
    vq, vs = quant_kv(v)
    ok = slots >= 0
    pages, off = (slots[ok] // kv.page_size).long(), (slots[ok] % kv.page_size).long()
    kq, vq, ks, vs = kq[ok], vq[ok], ks[ok], vs[ok]
    t, hk, d = kq.shape
    kv.k[pages, :, :, off] = kq.reshape(t, hk, d // 64, 64)
    vslot = torch.tensor(V_SLOT_OF_TOKEN, device=slots.device)[off]
    kv.v[pages, :, :, vslot] = vq
    kv.k_scale[pages, :, off] = ks
    kv.v_scale[pages, :, off] = vs

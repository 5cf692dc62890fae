"""Prefill (chunk) attention dispatch.

``run`` gathers each sequence's K/V rows of the chunk from the FP8 page pool and attends causally.  The
tcgen05 flash-attention kernel is used when the library exports it; otherwise the gathered rows go through
PyTorch's scaled-dot-product attention.
"""

from __future__ import annotations

import torch

from .lib import lib


def _gather(kv, slots: torch.Tensor):
    from .reference import gather_slots
    k, v = gather_slots(kv, slots)
    return k.to(torch.bfloat16), v.to(torch.bfloat16)  # [T, Hk, D]


def run(q: torch.Tensor, kv, step, *, n_kv: int, sm_scale: float) -> torch.Tensor:
    t, hq, d = q.shape
    out = torch.empty_like(q)
    k_all, v_all = _gather(kv, step.slots)
    native = hasattr(lib(), "mfq_attn_prefill_bf16") and d == 128
    for i in range(len(step.cu_seqlens) - 1):
        a, b = step.cu_seqlens[i], step.cu_seqlens[i + 1]
        if native:
            from .kernels import attn_prefill_bf16
            attn_prefill_bf16(q[a:b], k_all[a:b], v_all[a:b], sm_scale, out=out[a:b])
            continue
        qq = q[a:b].transpose(0, 1).unsqueeze(0)  # [1, Hq, T, D]
        kk = k_all[a:b].transpose(0, 1).unsqueeze(0)
        vv = v_all[a:b].transpose(0, 1).unsqueeze(0)
        o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=sm_scale, enable_gqa=True)
        out[a:b] = o.squeeze(0).transpose(0, 1)
    return out

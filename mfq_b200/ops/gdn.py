"""Gated DeltaNet operators: causal conv + SiLU, the gated delta-rule recurrence with fused gated RMSNorm, and the
state selection after an MTP verify window.  CUDA kernels on device tensors, a plain fp32 torch restatement on CPU
tensors (the oracle of the GPU tests; same math as ``mfq/kernels/gated_delta_net.py`` of the reference).

Layout: sequences form a regular ``[B, L]`` grid (decode ``L = 1``, verify ``L = K + 1``, prefill ``B = 1``); ``slot[b]``
names the row's state slot (``< 0`` skips the row).  ``conv_state [slots, 3, C]`` fp32 holds the last three pre-conv
inputs, ``state [slots, Hv, dk, dv]`` fp32 the delta-rule memory.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.nn.functional as F

from .lib import check, lib, ptr, stream_ptr

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_bound = False
PREFILL_MIN_TOKENS = 8  # rows longer than this take the prefill kernels
CHUNKED_MIN_TOKENS = 64  # rows at least this long take the chunked (WY) prefill; shorter ones the token-serial one
_scratch: dict[int, torch.Tensor] = {}


def _lib():
    global _bound
    L = lib()
    if not _bound:
        L.mfq_gdn_conv.argtypes = [_vp] * 6 + [_i] * 4 + [_vp]
        L.mfq_gdn_recurrent.argtypes = [_vp] * 11 + [_i] * 6 + [_f, _i, _i, _vp]
        L.mfq_gdn_select.argtypes = [_vp] * 6 + [_i] * 6 + [_vp]
        L.mfq_gdn_prefill.argtypes = [_vp] * 12 + [_i] * 6 + [_f, _i, _i, _vp]
        L.mfq_gdn_prefill_chunked.argtypes = [_vp] * 12 + [C.c_longlong] + [_i] * 6 + [_f, _i, _i, _vp, _vp]
        L.mfq_gdn_chunk_scratch_floats.argtypes = [_i] * 4
        L.mfq_gdn_chunk_scratch_floats.restype = C.c_longlong
        _bound = True
    return L


def conv(x: torch.Tensor, conv_state: torch.Tensor, w: torch.Tensor, slot: torch.Tensor, L: int,
         conv_ckpt: torch.Tensor | None = None) -> torch.Tensor:
    """``x [B*L, C]`` bf16 -> ``silu(causal_conv4(x))`` fp32; updates ``conv_state`` (or fills ``conv_ckpt [B, L, 3, C]``
    with the history after each token and leaves ``conv_state`` alone)."""
    n, c = x.shape
    b = n // L
    out = torch.empty((n, c), dtype=torch.float32, device=x.device)
    if x.is_cuda:
        check(_lib().mfq_gdn_conv(ptr(x), ptr(conv_state), ptr(w), ptr(slot), ptr(out), ptr(conv_ckpt), b, L, c, x.stride(0),
                                  stream_ptr()),
              "gdn_conv", 1 if conv_ckpt is not None else 2)
        return out
    xs = x.float().view(b, L, c)
    for r in range(b):
        s = int(slot[r])
        if s < 0:
            continue
        hist = torch.cat([conv_state[s], xs[r]], 0)  # [3 + L, C]
        for t in range(L):
            y = (hist[t : t + 4] * w.T).sum(0)
            out[r * L + t] = y * torch.sigmoid(y)
            if conv_ckpt is not None:
                conv_ckpt[r, t] = hist[t + 1 : t + 4]
        if conv_ckpt is None:
            conv_state[s] = hist[L : L + 3]
    return out


def recurrent(qkv: torch.Tensor, z: torch.Tensor, a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor,
              dt_bias: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, slot: torch.Tensor, L: int, Hk: int, Hv: int,
              eps: float = 1e-6, ckpt: torch.Tensor | None = None) -> torch.Tensor:
    """Gated delta rule over ``L`` tokens per row + gated RMSNorm; returns ``y [B*L, Hv*dv]`` bf16.  Updates ``state``
    in place, or -- with ``ckpt [B, L, Hv, dk, dv]`` -- writes the state after every token there instead."""
    n = qkv.shape[0]
    rows = n // L
    dk, dv = state.shape[2], state.shape[3]
    y = torch.empty((n, Hv * dv), dtype=torch.bfloat16, device=qkv.device)
    if qkv.is_cuda and ckpt is None and L >= CHUNKED_MIN_TOKENS:
        # 64-token chunks: a parallel pre-pass solves each chunk's triangular system, a scan carries the state
        # over the chunks on tensor cores (``csrc/gdn_chunk.cu``); ``qkv`` is left as it is
        lb = _lib()
        need = int(lb.mfq_gdn_chunk_scratch_floats(rows, L, Hk, Hv))
        dev = qkv.device.index or 0
        scratch = _scratch.get(dev)
        if scratch is None or scratch.numel() < need:
            scratch = _scratch[dev] = torch.empty(need, dtype=torch.float32, device=qkv.device)
        o_raw = torch.empty((n, Hv * dv), dtype=torch.float32, device=qkv.device)
        from .lib import Workspace
        check(lb.mfq_gdn_prefill_chunked(ptr(qkv), ptr(z), ptr(a), ptr(b), ptr(A_log), ptr(dt_bias), ptr(norm_w), ptr(state),
                                         ptr(slot), ptr(y), ptr(o_raw), ptr(scratch), scratch.numel(), rows, L, Hk, Hv, dk, dv,
                                         float(eps), z.stride(0), a.stride(0), ptr(Workspace.get(qkv.device).status),
                                         stream_ptr()), "gdn_prefill_chunked", 3)
        return y
    if qkv.is_cuda and ckpt is None and L > PREFILL_MIN_TOKENS:
        # long rows: pre-pass / 4-threads-per-column recurrence / post-pass (normalises q and k inside ``qkv`` in place)
        o_raw = torch.empty((n, Hv * dv), dtype=torch.float32, device=qkv.device)
        gates = torch.empty((n, Hv, 2), dtype=torch.float32, device=qkv.device)
        check(_lib().mfq_gdn_prefill(ptr(qkv), ptr(z), ptr(a), ptr(b), ptr(A_log), ptr(dt_bias), ptr(norm_w), ptr(state), ptr(slot),
                                     ptr(y), ptr(o_raw), ptr(gates), rows, L, Hk, Hv, dk, dv, float(eps), z.stride(0), a.stride(0),
                                     stream_ptr()), "gdn_prefill")
        return y
    if qkv.is_cuda:
        check(_lib().mfq_gdn_recurrent(ptr(qkv), ptr(z), ptr(a), ptr(b), ptr(A_log), ptr(dt_bias), ptr(norm_w), ptr(state),
                                       ptr(ckpt), ptr(slot), ptr(y), rows, L, Hk, Hv, dk, dv, float(eps), z.stride(0), a.stride(0),
                                       stream_ptr()),
              "gdn_recurrent")
        return y
    rep = Hv // Hk
    q = qkv[:, : Hk * dk].view(n, Hk, dk)
    k = qkv[:, Hk * dk : 2 * Hk * dk].view(n, Hk, dk)
    v = qkv[:, 2 * Hk * dk :].view(n, Hv, dv)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)  # [n, Hv, dk]
    decay = torch.exp(-torch.exp(A_log)[None] * F.softplus(a.float() + dt_bias[None]))  # [n, Hv]
    beta = torch.sigmoid(b.float())
    zz = z.float().view(n, Hv, dv)
    for r in range(rows):
        s_id = int(slot[r])
        if s_id < 0:
            continue
        S = state[s_id].clone()  # [Hv, dk, dv]
        for t in range(L):
            i = r * L + t
            S = S * decay[i][:, None, None]
            kv = (S * k[i][:, :, None]).sum(1)
            delta = (v[i] - kv) * beta[i][:, None]
            S = S + k[i][:, :, None] * delta[:, None, :]
            o = (S * q[i][:, :, None]).sum(1)  # [Hv, dv]
            o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w[None] * (zz[i] * torch.sigmoid(zz[i]))
            y[i] = o.reshape(-1).to(torch.bfloat16)
            if ckpt is not None:
                ckpt[r, t] = S
        if ckpt is None:
            state[s_id] = S
    return y


def select(ckpt: torch.Tensor, conv_ckpt: torch.Tensor, state: torch.Tensor, conv_state: torch.Tensor, slot: torch.Tensor,
           keep: torch.Tensor) -> None:
    """After a verify window: adopt the checkpoint of window position ``keep[b]`` as the row's state."""
    b, L, hv, dk, dv = ckpt.shape
    c = conv_ckpt.shape[-1]
    if ckpt.is_cuda:
        check(_lib().mfq_gdn_select(ptr(ckpt), ptr(conv_ckpt), ptr(state), ptr(conv_state), ptr(slot), ptr(keep), b, L, hv, dk,
                                    dv, c, stream_ptr()), "gdn_select")
        return
    for r in range(b):
        s = int(slot[r])
        if s >= 0:
            t = min(max(int(keep[r]), 0), L - 1)
            state[s] = ckpt[r, t]
            conv_state[s] = conv_ckpt[r, t]

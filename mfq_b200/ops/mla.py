"""Latent-attention (weight-absorbed MLA) operators over the shared-row FP8 cache: the row writer and the decode
attention (``csrc/mla_decode.cu``).  The cache is the generic paged cache with one KV head of width 576
(``[rotary key part 64 | normalised latent 512]``); a token's value is the latent part of its row."""

from __future__ import annotations

import ctypes as C

import torch

from .lib import Workspace, check, lib, ptr, stream_ptr

ROW_WIDTH, LATENT = 576, 512
_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_bound = False


def _lib():
    global _bound
    L = lib()
    if not _bound:
        L.mfq_mla_latent_write.argtypes = [_vp] * 6 + [_i, _vp]
        L.mfq_mla_decode.argtypes = [_vp] * 10 + [_i, _i, _i, _f, _i, _vp, _vp]
        _bound = True
    return L


def latent_write(rows: torch.Tensor, slots: torch.Tensor, kv) -> None:
    """``rows [T, 576]`` bf16 (rotary part already rotated) -> FP8 codes and one multiplier per token at ``slots``
    (``page * 16 + offset``; negative = skip) of one layer's pages."""
    t, d = rows.shape
    if d != ROW_WIDTH or kv.k.shape[-3] * kv.k.shape[-1] != ROW_WIDTH or kv.k.shape[-4] != 1:
        raise ValueError("the latent cache holds one 576-wide row per token")
    check(_lib().mfq_mla_latent_write(ptr(rows.contiguous()), ptr(slots), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale),
                                      t, stream_ptr()), "mla_latent_write")


def decode(q: torch.Tensor, kv, block_table: torch.Tensor, seq_lens: torch.Tensor, *, sm_scale: float, splits: int = 1,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """``q [B, H, 576]`` bf16 in cache-row space (``q_rope | W_k^T q_nope``) -> the latent mix ``[B, H, 512]`` bf16 of every
    head over the first ``seq_lens[b]`` cached rows of sequence ``b``."""
    b, h, d = q.shape
    if d != ROW_WIDTH:
        raise ValueError("queries must be 576 wide (rotary part | absorbed latent part)")
    out = torch.empty((b, h, LATENT), dtype=torch.bfloat16, device=q.device) if out is None else out
    ws = Workspace.get(q.device)
    splits = max(1, int(splits))
    if splits > 1 and (b * h * splits * LATENT > ws.attn_acc.numel() or b * h * splits * 2 > ws.attn_ml.numel()):
        splits = 1
    check(_lib().mfq_mla_decode(ptr(q.contiguous()), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale), ptr(block_table),
                                ptr(seq_lens), ptr(out), ptr(ws.attn_acc), ptr(ws.attn_ml), b, h, block_table.shape[1],
                                float(sm_scale), splits, ptr(ws.status), stream_ptr()), "mla_decode", 2 if splits > 1 else 1)
    return out

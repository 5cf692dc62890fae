"""4-bit group-quantized weights for the in-pipeline-decode GEMM (``csrc/w4_gemm.cu``): repacking and the call.

``w = s[n, g] * q[n, k] - b[n, g]`` with ``g = k // group_size`` -- exactly the NINT reconstruction for code widths
up to 4 bits (``s = d * ls``, ``b = dmin * lm``).  :func:`repack` turns codes + group parameters into the layout the
kernel streams: per (128-row tile, 64-wide K block) 4 KB of nibbles, rows contiguous, 8 codes per 32-bit word in the
order ``c0 c2 c4 c6 c1 c3 c5 c7`` (so one mask per nibble pair yields two bf16 values in memory order), and the
group parameters transposed to ``[tile, group, row]`` as ``bf16 s | bf16 -b``.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import kernels as K
from .lib import Workspace, check, lib, ptr, stream_ptr

TILE_N, BLOCK_K = 128, 64
_NIBBLE_COLUMN = np.array([0, 2, 4, 6, 1, 3, 5, 7])  # nibble n of a word holds column _NIBBLE_COLUMN[n] of its 8


@dataclass
class W4Weight:
    packed: torch.Tensor  # uint8 [n_tiles, k_blocks, 128, 32]
    group: torch.Tensor  # int32 [n_tiles, groups, 128]
    n: int
    k: int
    group_size: int
    kind: int = 0  # 0: affine codes (NINT), 1: MXFP4 (E2M1 codes, one power-of-two multiplier per 32 inputs)

    def to(self, device) -> "W4Weight":
        return W4Weight(self.packed.to(device), self.group.to(device), self.n, self.k, self.group_size, self.kind)

    @property
    def bits_per_weight(self) -> float:
        return 8.0 * (self.packed.numel() + 4 * self.group.numel()) / (self.n * self.k)


def _bf16_bits(x: np.ndarray) -> np.ndarray:
    return (torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16))


def repack(codes: np.ndarray, scale: np.ndarray, shift: np.ndarray, group_size: int) -> W4Weight:
    """``codes [N, K]`` (values 0..15), ``scale`` / ``shift`` ``[N, K / group_size]`` fp32 -> kernel layout."""
    n, k = codes.shape
    if k % BLOCK_K or group_size % 8 or k % group_size or codes.max(initial=0) > 15:
        raise ValueError("w4 repack needs K % 64 == 0, a group size that is a multiple of 8 and divides K, codes <= 15")
    groups = k // group_size
    n_pad = math.ceil(n / TILE_N) * TILE_N
    q = np.zeros((n_pad, k), dtype=np.uint32)
    q[:n] = codes
    s = np.zeros((n_pad, groups), dtype=np.float32)
    b = np.zeros((n_pad, groups), dtype=np.float32)
    s[:n], b[:n] = scale, shift
    words = q.reshape(n_pad, k // 8, 8)[:, :, _NIBBLE_COLUMN]  # [.., nibble] = code of the column that nibble holds
    word = (words << (4 * np.arange(8, dtype=np.uint32))[None, None, :]).sum(-1).astype("<u4")  # [n_pad, k/8]
    packed = word.reshape(n_pad // TILE_N, TILE_N, k // BLOCK_K, 8).transpose(0, 2, 1, 3)  # tile, kb, row, word
    packed = np.ascontiguousarray(packed).view(np.uint8).reshape(n_pad // TILE_N, k // BLOCK_K, TILE_N, 32)
    s_bits = _bf16_bits(s)
    bias_bits = _bf16_bits(-b)
    g = (s_bits.astype(np.uint32) | (bias_bits.astype(np.uint32) << 16)).reshape(n_pad // TILE_N, TILE_N, groups)
    g = np.ascontiguousarray(g.transpose(0, 2, 1)).view(np.int32)
    return W4Weight(torch.from_numpy(packed.copy()), torch.from_numpy(g.copy()), n, k, group_size)


def repack_torch(codes: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, group_size: int) -> W4Weight:
    """:func:`repack` with torch ops on the tensors' device (large matrices; same layout, same rounding)."""
    n, k = codes.shape
    if k % BLOCK_K or group_size % 8 or k % group_size:
        raise ValueError("w4 repack needs K % 64 == 0 and a group size that is a multiple of 8 and divides K")
    dev = codes.device
    groups = k // group_size
    n_pad = math.ceil(n / TILE_N) * TILE_N
    q = torch.zeros((n_pad, k), dtype=torch.int64, device=dev)
    q[:n] = codes.to(torch.int64)
    perm = torch.as_tensor(_NIBBLE_COLUMN, device=dev)
    words = q.view(n_pad, k // 8, 8)[:, :, perm]
    word = (words << (4 * torch.arange(8, device=dev))).sum(-1)  # < 2^32, held in int64
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    packed = word.view(n_pad // TILE_N, TILE_N, k // BLOCK_K, 8).permute(0, 2, 1, 3).contiguous()
    packed = packed.view(torch.uint8).view(n_pad // TILE_N, k // BLOCK_K, TILE_N, 32)
    s = torch.zeros((n_pad, groups), dtype=torch.float32, device=dev)
    b = torch.zeros((n_pad, groups), dtype=torch.float32, device=dev)
    s[:n], b[:n] = scale, shift
    s_bits = s.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    b_bits = (-b).to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    g = (s_bits | (b_bits << 16)).view(n_pad // TILE_N, TILE_N, groups).permute(0, 2, 1).contiguous()
    return W4Weight(packed, g, n, k, group_size)


def quantize_torch(w: torch.Tensor, group_size: int = 32) -> W4Weight:
    """Plain min/max 4-bit group quantization of a float matrix on its device (synthetic / benchmark weights; real
    checkpoints come through :func:`from_nint`, which keeps the NINT quantizer's least-squares fit)."""
    n, k = w.shape
    g = w.float().view(n, k // group_size, group_size)
    lo, hi = g.amin(-1), g.amax(-1)
    s = ((hi - lo) / 15.0).clamp_min(1e-12)
    codes = torch.round((g - lo[..., None]) / s[..., None]).clamp_(0, 15).to(torch.uint8).view(n, k)
    return repack_torch(codes, s, -lo, group_size)


_E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def from_mxfp4(t) -> W4Weight:
    """MXFP4 tensor (two E2M1 codes per byte, low nibble first; one E8M0 exponent per 32) -> :class:`W4Weight`."""
    rows, cols = t.shape
    if cols % BLOCK_K:
        raise ValueError("MXFP4 rows must be a multiple of 64 wide for the GEMM layout")
    raw = np.asarray(t.values, dtype=np.uint8).reshape(rows, cols // 2)
    codes = np.empty((rows, cols), dtype=np.uint8)
    codes[:, 0::2], codes[:, 1::2] = raw & 0xF, raw >> 4
    w = repack(codes, np.zeros((rows, cols // 32), np.float32), np.zeros((rows, cols // 32), np.float32), 32)
    e = np.zeros((w.packed.shape[0] * TILE_N, cols // 32), dtype=np.uint32)
    e[:rows] = np.asarray(t.scales, dtype=np.uint8).reshape(rows, cols // 32)
    g = (e << 7).reshape(-1, TILE_N, cols // 32).transpose(0, 2, 1)  # bf16 bits of 2^(e - 127) in the low half
    return W4Weight(w.packed, torch.from_numpy(np.ascontiguousarray(g).view(np.int32).copy()), rows, cols, 32, kind=1)


def from_nint(t) -> W4Weight:
    """NINT tensor (every row at most 4 code bits, 2-D, group size a multiple of 8) -> :class:`W4Weight`."""
    gs = t.spec.groupsize
    widths = t.q_widths() if hasattr(t, "q_widths") else np.full(t.q.shape[0], t.spec.bits)
    if int(np.max(widths)) > 4:
        raise ValueError("rows wider than 4 bits do not fit the 4-bit container")
    out, groups, _ = t.q.shape
    codes = t.q.reshape(out, groups * gs)[:, : t.neuron_len]
    if t.neuron_len != groups * gs:
        raise ValueError("row length must be a whole number of groups")
    scale = t.neuron_scale[:, None].astype(np.float32) * t.sub_scale.astype(np.float32)
    shift = t.neuron_min[:, None].astype(np.float32) * t.sub_min.astype(np.float32)
    return repack(codes, scale, shift, gs)


def concat_rows(parts: list[W4Weight]) -> W4Weight:
    """Stack weights along the output dimension (fused q|k|v, gate|up): every part but the last must hold a multiple
    of 128 rows, all parts the same K, group size and kind."""
    k, gs, kind = parts[0].k, parts[0].group_size, parts[0].kind
    if any((p.k, p.group_size, p.kind) != (k, gs, kind) for p in parts) or any(p.n % TILE_N for p in parts[:-1]):
        raise ValueError("parts do not stack: different geometry or a part that is not a whole number of 128-row tiles")
    return W4Weight(torch.cat([p.packed for p in parts], 0), torch.cat([p.group for p in parts], 0), sum(p.n for p in parts), k, gs, kind)


def from_checkpoint_tensor(t) -> W4Weight | None:
    """:class:`W4Weight` for a checkpoint tensor the 4-bit GEMM can run natively (2-D NINT with at most 4 code bits
    and a group size that is a multiple of 8, MXFP4, or MXFP4-SQ expanded to MXFP4), else None."""
    from ..formats.mx import MxTensor
    from ..formats.mxfp4sq import Mxfp4SqTensor, expanded
    from ..formats.nint import NintTensor
    if isinstance(t, Mxfp4SqTensor):
        t = expanded(t)  # palette-coded rows decode to legal E2M1 nibbles under E8M0 scales: the same kernel runs them
    try:
        if isinstance(t, NintTensor) and len(t.shape) == 2 and t.axis == 0:
            return from_nint(t)
        if isinstance(t, MxTensor) and t.dtype == "MXFP4":
            return from_mxfp4(t)
    except ValueError:
        return None
    return None


def dequantize(w: W4Weight) -> torch.Tensor:
    """fp32 ``[N, K]`` matrix exactly as the kernel's decode warps produce it (bf16-rounded values)."""
    packed = w.packed.cpu().numpy().view("<u4").reshape(w.packed.shape[0], w.packed.shape[1], TILE_N, 8)
    nib = (packed[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF  # [tile, kb, row, word, nibble]
    cols = np.empty_like(nib)
    cols[..., _NIBBLE_COLUMN] = nib
    q = cols.transpose(0, 2, 1, 3, 4).reshape(w.packed.shape[0] * TILE_N, -1).astype(np.float32)  # [n_pad, K]
    g = w.group.cpu().numpy().view(np.uint32).transpose(0, 2, 1).reshape(-1, w.group.shape[1])
    if w.kind == 1:
        s = torch.from_numpy((g & 0xFFFF).astype(np.int16)).view(torch.bfloat16).float().repeat_interleave(32, 1)
        return (torch.from_numpy(_E2M1[q.astype(np.int64)]) * s)[: w.n]
    s = torch.from_numpy((g & 0xFFFF).astype(np.int16)).view(torch.bfloat16).float()
    bias = torch.from_numpy((g >> 16).astype(np.int16)).view(torch.bfloat16).float()
    s, bias = s.repeat_interleave(w.group_size, 1), bias.repeat_interleave(w.group_size, 1)
    val = torch.addcmul(bias.double(), s.double(), torch.from_numpy(q).double())  # s * q - b, one rounding like the FMA
    return val.float().to(torch.bfloat16).float()[: w.n]


def w4_gemm(x: torch.Tensor, w: W4Weight, *, residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
            token_tile: int | None = None, splits: int | None = None) -> torch.Tensor:
    """``x [M, K]`` bf16 -> ``x @ W^T (+ residual)`` bf16 ``[M, N]`` with the weights decoded inside the GEMM pipeline."""
    m, k = x.shape
    if not x.is_cuda:
        y = x.float() @ dequantize(w).T
        if residual is not None:
            y = y + residual.float()
        return y.to(torch.bfloat16)
    out = torch.empty((m, w.n), dtype=torch.bfloat16, device=x.device) if out is None else out
    bt = token_tile or K._token_tile(m)
    sp = K.pick_splits(m, w.n, k // 2) if splits is None else splits  # K blocks are 64 wide here: same work model
    ws = Workspace.get(x.device)
    fn = lib().mfq_w4_gemm
    fn.argtypes = [C.c_void_p] * 6 + [C.c_size_t, C.c_void_p, C.c_int, C.c_void_p] + [C.c_int] * 7 + [C.c_void_p]
    rc = fn(ptr(w.packed), ptr(w.group), ptr(x), ptr(out), ptr(residual), ptr(ws.splitk), ws.splitk.numel(), ptr(ws.counters),
            ws.counters.numel(), ptr(ws.status), m, w.n, k, w.group_size, bt, sp, w.kind, stream_ptr())
    check(rc, "w4_gemm")
    return out

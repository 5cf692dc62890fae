"""NINT8-1: activations in 32-value blocks of int8 codes with an FP16 step and an FP16 block sum -- the layout of
llama.cpp's Q8_1 activation blocks.  It is not a weight format; it exists so that an evaluation can put the SAME
activation rounding in front of a product as a llama.cpp run does and attribute the remaining divergence to the weights.

    amax = max |x| over the block      step = amax / 127 (FP32)      q = clamp(round_half_away(x / step), -127, 127)
    d = fp16(step)      s = fp16(sum(q) * step)      reconstruction = fp16(q * fp32(d))

:func:`quantize_nint8_one` restates ``mfq/formats/nint8_one.py:33-64`` of the reference in NumPy;
:func:`fake_quantize_nint8_one` is the same rounding on a torch tensor (any device), returning only the reconstruction.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BLOCK = 32
QMAX = 127


@dataclass(frozen=True)
class Nint8OneBlocks:
    q: np.ndarray              # [..., blocks, 32] int8
    d: np.ndarray              # [..., blocks] float16 step
    s: np.ndarray              # [..., blocks] float16 sum(q) * step
    reconstructed: np.ndarray  # [..., width] float16


def quantize_nint8_one(values) -> Nint8OneBlocks:
    x = np.asarray(values, dtype=np.float32)
    if x.ndim < 1 or x.size == 0:
        raise ValueError("NINT8-1 needs a non-empty array")
    if not np.isfinite(x).all():
        raise ValueError("NINT8-1 needs finite values")
    width = x.shape[-1]
    blocks = -(-width // BLOCK)
    pad = np.zeros(x.shape[:-1] + (blocks * BLOCK,), dtype=np.float32)
    pad[..., :width] = x
    g = pad.reshape(x.shape[:-1] + (blocks, BLOCK))
    step = np.abs(g).max(-1) / np.float32(QMAX)
    inv = np.divide(np.float32(1.0), step, out=np.zeros_like(step), where=step != 0)
    scaled = g * inv[..., None]
    q = np.clip(np.where(scaled >= 0, np.floor(scaled + np.float32(0.5)), np.ceil(scaled - np.float32(0.5))), -QMAX, QMAX).astype(np.int8)
    d = step.astype(np.float16)
    s = (q.astype(np.int32).sum(-1).astype(np.float32) * step).astype(np.float16)
    rec = (q.astype(np.float32) * d.astype(np.float32)[..., None]).astype(np.float16)
    return Nint8OneBlocks(q, d, s, rec.reshape(x.shape[:-1] + (blocks * BLOCK,))[..., :width].copy())


def fake_quantize_nint8_one(x):
    """torch tensor -> the FP16 reconstruction of its NINT8-1 blocks along the last axis (same shape, same device)."""
    import torch
    width = x.shape[-1]
    blocks = -(-width // BLOCK)
    g = torch.nn.functional.pad(x.float(), (0, blocks * BLOCK - width)).reshape(x.shape[:-1] + (blocks, BLOCK))
    step = g.abs().amax(-1) / QMAX
    inv = torch.where(step != 0, 1.0 / step, torch.zeros_like(step))
    scaled = g * inv[..., None]
    q = torch.where(scaled >= 0, torch.floor(scaled + 0.5), torch.ceil(scaled - 0.5)).clamp(-QMAX, QMAX)
    rec = (q * step.half().float()[..., None]).half()
    return rec.reshape(x.shape[:-1] + (blocks * BLOCK,))[..., :width].contiguous()

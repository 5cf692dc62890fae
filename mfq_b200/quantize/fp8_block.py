"""bf16/fp32 -> block-scaled FP8: E4M3 codes with one fp32 multiplier per 128x128 block.

``scale = amax(block) / 448`` and ``code = rne_e4m3(x / scale)``.  The reference
re-quantizes only checkpoints that are already FP8 (``mfq/quantize/fp8_sq.py:137``);
this encoder produces the lossless all-SQ8 ``FP8-128SQ`` profile from higher precision.
Activations use the same E4M3 grid with one multiplier per token per 128 inputs
(:func:`quantize_act_1x128`), the pairing the tensor-core GEMM expects.
"""

from __future__ import annotations

import numpy as np
import torch

from ..formats.fp8sq import Fp8SqTensor, block_fp8_tensor

E4M3_MAX = 448.0

__all__ = ["quantize_fp8_block", "quantize_fp8_block_torch", "quantize_act_1x128", "dequantize_fp8_block_torch"]


def quantize_fp8_block_torch(w: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """``[rows, cols]`` -> (``float8_e4m3fn [rows, cols]``, fp32 scales ``[ceil(rows/b), ceil(cols/b)]``)."""
    rows, cols = w.shape
    pr, pc = (-rows) % block, (-cols) % block
    x = torch.nn.functional.pad(w.to(torch.float32), (0, pc, 0, pr))
    R, C = x.shape
    tiles = x.reshape(R // block, block, C // block, block)
    amax = tiles.abs().amax(dim=(1, 3))
    scale = (amax / E4M3_MAX).clamp_min(1e-12)
    q = (tiles / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(R, C)[:rows, :cols].contiguous(), scale.contiguous()


def dequantize_fp8_block_torch(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    rows, cols = q.shape
    s = scale.repeat_interleave(block, 0)[:rows].repeat_interleave(block, 1)[:, :cols]
    return q.to(torch.float32) * s


def quantize_act_1x128(x: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token, per-128-input activation quantization: returns (fp8 ``[M, K]``, fp32 ``[M, K/128]``)."""
    m, k = x.shape
    g = x.to(torch.float32).reshape(m, k // block, block)
    scale = (g.abs().amax(-1) / E4M3_MAX).clamp_min(1e-12)
    q = (g / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(m, k), scale


def quantize_fp8_block(weight, device: str | torch.device = "cpu") -> Fp8SqTensor:
    w = torch.as_tensor(np.asarray(weight, dtype=np.float32) if not torch.is_tensor(weight) else weight).to(device)
    q, s = quantize_fp8_block_torch(w)
    return block_fp8_tensor(q.view(torch.uint8).cpu().numpy(), s.cpu().numpy())

"""bf16/fp32 -> MXFP4 encoder (E2M1 elements, one E8M0 scale per 32 inputs).

The reference only carries natively-trained MXFP4 through its converter and has no
encoder from higher precision; this one exists so that random-init checkpoints can
be produced in the named format.  Scale choice follows the OCP MX rule
``e = floor(log2(amax)) - 2`` (E2M1's largest exponent is 2), refined by trying
``e`` and ``e + 1`` and keeping the lower squared error; elements round to the
nearest E2M1 value, ties to the even code.
"""

from __future__ import annotations

import numpy as np
import torch

from ..formats.mx import MXFP4_DTYPE, MxTensor

_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_EDGES = (_GRID[1:] + _GRID[:-1]) / 2  # decision thresholds between neighbouring codes

__all__ = ["quantize_mxfp4", "quantize_mxfp4_torch"]


def _round_e2m1(mag: torch.Tensor) -> torch.Tensor:
    """Magnitude (already divided by the block scale) -> 3-bit code, ties to even code."""
    edges = _EDGES.to(mag.device)
    code = torch.bucketize(mag, edges, right=False)  # mag == edge falls to the lower code
    tie = mag == edges[(code).clamp(max=6)]
    code = torch.where(tie & (code % 2 == 1), code + 1, code)
    return code.clamp(max=7)


def quantize_mxfp4_torch(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[rows, cols]`` float -> (packed nibbles ``[rows, cols/2]`` uint8, E8M0 ``[rows, cols/32]`` uint8)."""
    rows, cols = w.shape
    if cols % 32:
        raise ValueError("MXFP4 needs a multiple of 32 columns")
    x = w.to(torch.float32).reshape(rows, cols // 32, 32)
    amax = x.abs().amax(-1)
    e0 = torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - 2
    grid = _GRID.to(w.device)
    best = None
    for bump in (0, 1):
        e = (e0 + bump).clamp(-127, 127)
        scale = torch.exp2(e)[..., None]
        code = _round_e2m1((x.abs() / scale).clamp(max=6.0))
        err = ((grid[code] * scale - x.abs()) ** 2).sum(-1)
        if best is None:
            best = (err, e, code)
        else:
            take = err < best[0]
            best = (torch.where(take, err, best[0]), torch.where(take, e, best[1]), torch.where(take[..., None], code, best[2]))
    _, e, code = best
    e = torch.where(amax > 0, e, torch.full_like(e, -127.0))
    nib = (code | ((x < 0).to(code.dtype) << 3)).to(torch.uint8).reshape(rows, cols)
    packed = nib[:, 0::2] | (nib[:, 1::2] << 4)
    return packed.contiguous(), (e + 127).to(torch.uint8).contiguous()


def quantize_mxfp4(weight, device: str | torch.device = "cpu") -> MxTensor:
    w = torch.as_tensor(np.asarray(weight, dtype=np.float32) if not torch.is_tensor(weight) else weight).to(device)
    packed, scales = quantize_mxfp4_torch(w)
    return MxTensor(MXFP4_DTYPE, tuple(w.shape), packed.cpu().numpy(), scales.cpu().numpy())

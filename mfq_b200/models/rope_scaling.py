"""YaRN context extension of rotary embeddings.

A model trained on ``original_max_position`` tokens runs on ``factor`` times that many by slowing down only the rotary
frequencies that would leave the trained range: dimension pair ``i`` of ``rot / 2`` keeps its frequency when it turns
more than ``beta_fast`` times inside the trained context (ramp 0), is divided by ``factor`` when it turns less than
``beta_slow`` times (ramp 1), and is blended linearly in between.  cos / sin are multiplied by the attention factor
``0.1 ln(factor) + 1`` (so the logits grow by its square), which keeps the softmax temperature of the longer context.

The kernel evaluates the same closed form per rotary pair (``rope_kv_write`` with the four numbers of
:meth:`YarnScaling.kernel_args`); :func:`mfq_b200.ops.reference.rope` takes the table of :meth:`YarnScaling.inv_freq`.
Reference: ``cpp_runtime/core/include/mfq/yarn.h`` and the runtime flag ``--yarn-context-extension``
(``cpp_runtime/backends/cuda/commands/cli.h:126-195``); the Hugging Face ``rope_scaling`` keys are the import format.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass

import torch


@dataclass(frozen=True)
class YarnScaling:
    factor: float = 1.0
    original_max_position: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    attention_factor: float | None = None  # None: 0.1 ln(factor) + 1
    truncate: bool = True  # round the correction range outwards to whole pair indices
    softmax_scale_factor: float = 1.0  # extra factor on the attention scale (latent-attention models: mscale_all_dim squared)

    # ---- import / export ---------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict | None) -> "YarnScaling | None":
        if not d:
            return None
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_hf(cls, hf_config: dict) -> "YarnScaling | None":
        """``rope_scaling`` of a Hugging Face ``config.json`` (``rope_type`` / ``type`` = ``yarn``), else None."""
        rs = hf_config.get("rope_scaling") or hf_config.get("rope_parameters") or {}
        if (rs.get("rope_type") or rs.get("type")) != "yarn":
            return None
        factor = float(rs["factor"])
        original = int(rs.get("original_max_position_embeddings") or
                       round(hf_config.get("max_position_embeddings", 4096) / factor))
        att = rs.get("attention_factor")
        if att is None and rs.get("mscale") and rs.get("mscale_all_dim"):
            def ms(scale, m):
                return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
            att = ms(factor, float(rs["mscale"])) / ms(factor, float(rs["mscale_all_dim"]))
        soft = 1.0
        if hf_config.get("kv_lora_rank") and rs.get("mscale_all_dim"):  # these models also raise the softmax scale
            m = 0.1 * float(rs["mscale_all_dim"]) * math.log(factor) + 1.0 if factor > 1 else 1.0
            soft = m * m
        return cls(factor=factor, original_max_position=original, beta_fast=float(rs.get("beta_fast") or 32.0),
                   beta_slow=float(rs.get("beta_slow") or 1.0), attention_factor=None if att is None else float(att),
                   truncate=bool(rs.get("truncate", True)), softmax_scale_factor=soft)

    # ---- the numbers -------------------------------------------------------------------------------------------------
    @property
    def mscale(self) -> float:
        if self.attention_factor is not None:
            return float(self.attention_factor)
        return 1.0 if self.factor <= 1.0 else 0.1 * math.log(self.factor) + 1.0

    def correction_range(self, rot: int, theta: float) -> tuple[float, float]:
        """Pair indices (low, high) between which the blend ramps from "keep" to "divide by factor"."""
        def dim_for(rotations: float) -> float:
            return rot * math.log(self.original_max_position / (rotations * 2 * math.pi)) / (2 * math.log(theta))
        low, high = dim_for(self.beta_fast), dim_for(self.beta_slow)
        if self.truncate:
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, rot - 1)
        if low == high:
            high += 0.001
        return float(low), float(high)

    def kernel_args(self, rot: int, theta: float) -> tuple[float, float, float, float]:
        """(factor, low, high, mscale) as the rotary kernel takes them."""
        low, high = self.correction_range(rot, theta)
        return float(self.factor), low, high, self.mscale

    def inv_freq(self, rot: int, theta: float, device=None) -> torch.Tensor:
        """fp32 ``[rot / 2]`` angular frequencies after the blend."""
        i = torch.arange(rot // 2, device=device, dtype=torch.float32)
        base = torch.exp2(-math.log2(theta) * (2 * i) / rot)
        if self.factor == 1.0:
            return base
        low, high = self.correction_range(rot, theta)
        ramp = ((i - low) / (high - low)).clamp(0.0, 1.0)
        return base * ((1.0 - ramp) + ramp / self.factor)

    def max_position(self) -> int:
        return int(self.original_max_position * self.factor)

"""Quantizers: float weights -> family tensors of :mod:`mfq_b200.formats`."""

from .expertwise import (DEFAULT_MIX_SEED, ExpertProfile, balanced_expert_mix, parse_profiles, quantize_expertwise,
                         quantize_matrix)
from .fp8_block import quantize_act_1x128, quantize_fp8_block, quantize_fp8_block_torch
from .mxfp4 import quantize_mxfp4, quantize_mxfp4_torch
from .nint import quantize_nint
from .nvq import quantize_nvq

"""GPU operators (hand-written sm_100a kernels behind a C ABI) and their PyTorch references."""

from . import reference
from .kernels import (argmax, decode_advance, embed, fp8_gemm, paged_attn_decode, quant_rows, rmsnorm_quant,
                      rope_kv_write, silu_mul_quant)
from .kernels import attn_prefill
from .kernels import ACT_NORM, ACT_PLAIN, ACT_SWIGLU, act_gemv_ok, act_gemv_pays, fp8_gemv_act
from .lib import Workspace, available, count_launches, launch_count

__all__ = ["reference", "argmax", "decode_advance", "embed", "fp8_gemm", "paged_attn_decode", "quant_rows",
           "rmsnorm_quant", "rope_kv_write", "silu_mul_quant", "Workspace", "available", "attn_prefill", "count_launches", "launch_count"]

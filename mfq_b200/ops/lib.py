"""ctypes binding of the in-tree CUDA library.

The library is required on a machine with a GPU: :func:`lib` raises if it is missing instead of falling
back to an eager PyTorch path, so a deployment never runs unfused by accident.  Workspaces (split-K
partials, tile counters, attention partials, the device status word) are allocated once per device and
reused by every call on that device's current stream.
"""

from __future__ import annotations

import ctypes as C
from functools import lru_cache

import torch

from .build import LIB_PATH

_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t

_SIGNATURES = {
    "mfq_fp8_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "mfq_fp8_gemm_pair": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "mfq_fp8_gemm_allreduce": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp,
                               _vp, _sz, _i, _vp],
    "mfq_fp8_gemm_allgather": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp],
    "mfq_peer_barrier": [_i, _i, _vp, _vp, _vp, _vp],
    "mfq_argmax_allgather": [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp],
    "mfq_rmsnorm_quant": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp],
    "mfq_quant_rows": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "mfq_kv_gather_dequant": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "mfq_attn_prefill_past": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp],
    "mfq_silu_mul_bf16": [_vp, _vp, _i, _i, _i, _vp],
    "mfq_gate_quant_rows": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "mfq_rope_kv_write_ex": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _f, _i, _vp],
    "mfq_rope_kv_write_yarn": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _f, _i,
                               _f, _f, _f, _f, _vp],
    "mfq_rope_kv_write": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp],
    
    "mfq_paged_attn_decode_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp],
    "mfq_argmax": [_vp, _vp, _i, _i, _i, _vp],
    "mfq_embed": [_vp, _vp, _vp, _i, _i, _vp],
    "mfq_decode_advance": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp],
    "mfq_mtp_prepare": [_vp] * 9 + [_i, _i, _i, _i, _vp],
    "mfq_mtp_accept": [_vp] * 10 + [_i, _i, _vp],
    "mfq_mtp_select_rows": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "mfq_nvq_assign": [_vp, _vp, _vp, _vp, _vp, C.c_longlong, _i, _i, _vp],
    "mfq_fp8_gemv": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "mfq_fp8_gemv_act": [_vp, _vp, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _i, _vp],
    "mfq_fp8_gemv_grouped": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp],
    "mfq_attn_prefill_d256": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp, _vp],
    "mfq_attn_prefill_bf16": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp, _vp],
}


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH.name} is not built; run `python -m mfq_b200.ops.build` (needs nvcc) before using GPU ops")
    handle = C.CDLL(str(LIB_PATH))
    for name, argtypes in _SIGNATURES.items():
        if hasattr(handle, name):
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = C.c_int
    return handle


def available() -> bool:
    return LIB_PATH.exists() and torch.cuda.is_available()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# the wait on another rank that ran out, as tagged by the kernels (status word bits 8 and up)
_PEER_WAIT_SITES = {1: "all-gather GEMM: shard flag", 2: "GEMM all-reduce epilogue: tile flags", 3: "expert all-to-all: dispatched rows", 10: "expert all-to-all: combined rows",
                    4: "arg-max all-gather", 5: "row all-reduce", 6: "peer barrier", 7: "row all-gather",
                    8: "fused reduce: partials ready", 9: "fused reduce: rows pushed"}


class Workspace:
    """Per-device scratch shared by the kernels (sized once; grows never during graph capture)."""

    _by_device: dict[int, "Workspace"] = {}

    def __init__(self, device: torch.device, splitk_bytes: int = 64 << 20, counters: int = 1 << 16,
                 attn_floats: int = 16 << 20) -> None:
        self.device = device
        self.splitk = torch.empty(splitk_bytes, dtype=torch.uint8, device=device)
        self.counters = torch.zeros(counters, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.attn_acc = torch.empty(attn_floats, dtype=torch.float32, device=device)
        self.attn_ml = torch.empty(attn_floats // 32, dtype=torch.float32, device=device)

    @classmethod
    def get(cls, device: torch.device) -> "Workspace":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        ws = cls._by_device.get(idx)
        if ws is None:
            ws = cls(torch.device("cuda", idx))
            cls._by_device[idx] = ws
        return ws

    def check(self) -> None:
        """Raise if any kernel recorded a timed-out wait since the last check (synchronizes)."""
        word = int(self.status[0].item())
        if word:
            detail = self.status[1:].tolist()
            self.status.zero_()
            code, site = word & 0xFF, word >> 8
            where = f", wait site {site} ({_PEER_WAIT_SITES.get(site, '?')}; detail {detail})" if site else ""
            raise RuntimeError(f"a kernel gave up waiting (status code {code}{where}); results are invalid")


_LAUNCHES = [0]
_COUNTING = [False]


def count_launches(enable: bool) -> None:
    """Turn on counting of kernel launches issued through this module (used by the benchmark)."""
    _COUNTING[0] = bool(enable)


def launch_count() -> int:
    return _LAUNCHES[0]


def check(rc: int, what: str, launches: int = 1) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed on the host side with code {rc}")
    if _COUNTING[0]:
        _LAUNCHES[0] += launches

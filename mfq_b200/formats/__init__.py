"""Byte-level codecs of the ``.mfq`` checkpoint container and its tensor families."""

from .container import (ASSET_DTYPE, ASSET_PREFIX, MFQ_MAGIC, FileHeader, MfqStore, TensorRecord, canonical_dtype,
                        load, open_mfq, pack_tensor, save, save_sharded, shard_paths, unpack_tensor, write_streaming)
from .dense import Bf16Array, Fp8E4M3Array, from_bf16, to_bf16
from .fp8sq import FP8_128SQ_DTYPE, MXFP8_SQ_DTYPE, Fp8SqTensor, block_fp8_tensor, dequantize_fp8sq
from .mfe import MfePool, MfeTensor
from .mx import MXFP4_DTYPE, MXFP8_DTYPE, MxTensor, dequantize_mx
from .mxfp4sq import MXFP4_SQ_DTYPE, Mxfp4SqTensor
from .nint import NINT_DTYPE, NintSpec, NintTensor, dequantize_nint
from .nvq import NVQ_DTYPE, NvqJscTensor, NvqSpec, NvqTensor, dequantize_nvq


def dequantize(t):
    """Any family tensor -> float32 ndarray in its logical shape."""
    import numpy as np
    from . import mxfp4sq as _sq
    from .npq0 import Npq0Tensor, dequantize_npq0
    if isinstance(t, Npq0Tensor):
        return dequantize_npq0(t)
    from .nvq1 import Nvq1Tensor, dequantize_nvq1
    if isinstance(t, Nvq1Tensor):
        return dequantize_nvq1(t)
    from .nepq import NepqTensor, dequantize_nepq
    if isinstance(t, NepqTensor):
        return dequantize_nepq(t)  # logical coordinates: a rotation is undone
    from .nint8zero import Nint8ZeroTensor, dequantize_nint8_zero
    if isinstance(t, Nint8ZeroTensor):
        return dequantize_nint8_zero(t)
    if isinstance(t, NintTensor):
        return dequantize_nint(t)
    if isinstance(t, (NvqTensor, NvqJscTensor)):
        return dequantize_nvq(t)
    if isinstance(t, MxTensor):
        return dequantize_mx(t)
    if isinstance(t, Fp8SqTensor):
        return dequantize_fp8sq(t)
    if isinstance(t, Mxfp4SqTensor):
        return _sq.dequantize_mxfp4sq(t)
    if isinstance(t, MfeTensor):
        n, out, k = t.shape
        full = np.empty((n, out, k), dtype=np.float32)
        for pool in t.pools:
            rows = dequantize(pool.tensor).reshape(len(pool.expert_ids), out, k)
            full[np.asarray(pool.expert_ids)] = rows
        return full
    if isinstance(t, Bf16Array):
        return from_bf16(t)
    if isinstance(t, Fp8E4M3Array):
        from .mx import e4m3_to_float
        return e4m3_to_float(np.asarray(t))
    return np.asarray(t, dtype=np.float32)

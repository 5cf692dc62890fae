"""MFE ("mixed-format experts"): one logical ``[experts, out, in]`` tensor stored as pools.

Each pool groups experts that share one family/spec; its payload is that family's
blob over the stacked ``[pool_experts * out, in]`` matrix.  Pools must cover every
expert exactly once.  Layout parity: ``mfq/formats/io.py:486-494,723-760,797-848``.

    "MFE1" u32 n_experts, out_per_expert, neuron_len, pool_count
    per pool: u32 expert_count, u32 dtype_nbytes(<=32), u64 payload_nbytes, u64 runtime_nbytes
              i32 expert_ids[expert_count], ascii dtype, runtime payload, tensor payload
"""

from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Any, Callable

import numpy as np

_HEAD = struct.Struct("<4sIIII")
_POOL = struct.Struct("<IIQQ")
_MAGIC = b"MFE1"


@dataclass
class MfePool:
    expert_ids: np.ndarray  # int32, ascending not required
    tensor: Any  # a family tensor over [len(expert_ids) * out, in]
    runtime: bytes = b""


@dataclass
class MfeTensor:
    shape: tuple[int, int, int]  # (experts, out_per_expert, neuron_len)
    pools: tuple[MfePool, ...]

    def __post_init__(self) -> None:
        ids = np.concatenate([np.asarray(p.expert_ids, dtype=np.int64).reshape(-1) for p in self.pools]) if self.pools else np.empty(0, np.int64)
        if ids.size != self.shape[0] or not np.array_equal(np.sort(ids), np.arange(self.shape[0])):
            raise ValueError("MFE pools must cover every expert exactly once")

    def expert_location(self) -> dict[int, tuple[int, int]]:
        """expert id -> (pool index, position inside the pool)."""
        where = {}
        for pi, p in enumerate(self.pools):
            for pos, e in enumerate(np.asarray(p.expert_ids).reshape(-1)):
                where[int(e)] = (pi, pos)
        return where


_ROTATION = struct.Struct("<4sIIQ")


def rotation_runtime(tensor) -> bytes:
    """The runtime record of a pool whose tensor is a rotated NEPQ cohort: ``"HSG1" u32 K, u32 block, u64 seed`` and the
    +-1 diagonal as K int8 values, so that a runtime can rotate activations without deriving the diagonal
    (``mfq/formats/io.py:675-696`` of the reference); empty for every other pool."""
    from .nepq import NepqTensor, rotation_signs
    if not isinstance(tensor, NepqTensor) or not tensor.rotation_block:
        return b""
    k = int(tensor.shape[2])
    return _ROTATION.pack(b"HSG1", k, int(tensor.rotation_block), int(tensor.rotation_seed)) + \
        rotation_signs(k, tensor.rotation_block, tensor.rotation_seed).tobytes()


def pack_mfe(t: MfeTensor, pack_tensor: Callable[[Any], tuple[str, bytes]]) -> bytes:
    n, out, k = t.shape
    parts = [_HEAD.pack(_MAGIC, n, out, k, len(t.pools))]
    for p in t.pools:
        if isinstance(p.tensor, MfeTensor):
            raise TypeError("MFE pools cannot nest")
        ids = np.ascontiguousarray(p.expert_ids, dtype="<i4").reshape(-1)
        dtype, payload = pack_tensor(p.tensor)
        name = dtype.encode("ascii")
        if not 0 < len(name) <= 32:
            raise ValueError(f"invalid MFE pool dtype {dtype!r}")
        runtime = p.runtime or rotation_runtime(p.tensor)
        parts += [_POOL.pack(ids.size, len(name), len(payload), len(runtime)), ids.tobytes(), name, runtime, payload]
    return b"".join(parts)


def unpack_mfe(blob, unpack_tensor: Callable[[str, Any], Any]) -> MfeTensor:
    magic, n, out, k, pool_count = _HEAD.unpack_from(blob, 0)
    if magic != _MAGIC:
        raise ValueError(f"bad MFE magic {magic!r}")
    off = _HEAD.size
    pools = []
    for _ in range(pool_count):
        if off + _POOL.size > len(blob):
            raise ValueError("truncated MFE pool header")
        count, dlen, plen, rlen = _POOL.unpack_from(blob, off)
        off += _POOL.size
        if count == 0 or not 0 < dlen <= 32 or off + 4 * count + dlen + rlen + plen > len(blob):
            raise ValueError("invalid or truncated MFE pool")
        ids = np.frombuffer(blob, dtype="<i4", count=count, offset=off).astype(np.int32)
        off += 4 * count
        dtype = bytes(blob[off : off + dlen]).decode("ascii")
        off += dlen
        runtime = bytes(blob[off : off + rlen])
        off += rlen
        tensor = unpack_tensor(dtype, memoryview(blob)[off : off + plen])
        off += plen
        if isinstance(tensor, MfeTensor):
            raise ValueError("nested MFE pool")
        if runtime[:4] == b"HSG1" and runtime != rotation_runtime(tensor):
            raise ValueError("MFE pool: the rotation record does not match its NEPQ tensor")
        pools.append(MfePool(ids, tensor, runtime))
    if off != len(blob):
        raise ValueError(f"MFE blob has {len(blob) - off} trailing bytes")
    return MfeTensor((n, out, k), tuple(pools))

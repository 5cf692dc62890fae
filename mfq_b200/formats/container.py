"""The ``.mfq`` container: header, record table, back-to-back blobs.

File layout (little endian; parity with ``mfq/formats/io.py:1019-1058`` and
``mfq/formats/header.py:15-27`` of the reference)::

    "MFQ1"  u32 version  str arch
    [version >= 2]  u32 n_extra, n_extra x (str key, str json_value)
    u32 n_tensors,  n_tensors x (str name, str dtype, u64 blob_nbytes)
    blobs in record order, no padding         (str = u32 length + utf-8 bytes)

The reader maps the file and decodes a tensor only when it is asked for, so a
multi-hundred-GB checkpoint opens in milliseconds and each tensor-parallel rank
touches only the bytes of its own shards.  Multi-file checkpoints
(``name-00001-of-0000N.mfq``) are opened as one logical store.
"""

from __future__ import annotations

import json
import mmap
import os
import re
import struct
from collections.abc import Iterator, Mapping
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import numpy as np

from . import fp8sq, mfe, mx, mxfp4sq, nepq, nint, nint8zero, npq0, nvq, nvq1
from .dense import DENSE_DTYPES, pack_dense, unpack_dense

MFQ_MAGIC = b"MFQ1"
ASSET_DTYPE = "BLOB"
ASSET_PREFIX = "__mfq_asset__/"
MFE_DTYPE = "MFE"

_OLD_NVQ = {"NIQ2", "NIQ2J", "NIQ3", "NVQ2", "NVQ2J", "NVQ2J-L", "NVQ2J-XL", "NVQ3", "NVQ3J", "NVQ3J-512", "NVQ3J-L"}
_SHARD_RE = re.compile(r"^(?P<stem>.+)-(?P<index>\d{5})-of-(?P<count>\d{5})\.mfq$")

__all__ = [
    "MFQ_MAGIC", "ASSET_DTYPE", "ASSET_PREFIX", "FileHeader", "TensorRecord", "MfqStore", "save", "load",
    "open_mfq", "pack_tensor", "unpack_tensor", "canonical_dtype", "write_streaming", "save_sharded", "shard_paths",
]


def canonical_dtype(dtype: str) -> str:
    """Map historical record spellings to family names (``NINT4`` -> ``NINT`` ...)."""
    if dtype == "NINTv2" or (len(dtype) == 5 and dtype.startswith("NINT") and dtype[4] in "12345678"):
        return nint.NINT_DTYPE
    if dtype == "NINTM":
        return MFE_DTYPE
    if dtype in _OLD_NVQ:
        return nvq.NVQ_DTYPE
    if dtype in ("MXFP4-SQ2", "MXFP4-SQ3"):
        return mxfp4sq.MXFP4_SQ_DTYPE
    return dtype


@dataclass
class FileHeader:
    version: int = 2
    model_arch: str = ""
    extra: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: str
    offset: int  # absolute byte offset inside its file
    nbytes: int
    file_index: int = 0


def pack_tensor(t) -> tuple[str, bytes]:
    """Tensor object -> (public dtype string, self-describing payload)."""
    if isinstance(t, (bytes, bytearray, memoryview)):
        return ASSET_DTYPE, bytes(t)
    if isinstance(t, mx.MxTensor):
        return t.dtype, mx.pack_mx(t)
    if isinstance(t, mxfp4sq.Mxfp4SqTensor):
        return mxfp4sq.MXFP4_SQ_DTYPE, mxfp4sq.pack_mxfp4sq(t)
    if isinstance(t, fp8sq.Fp8SqTensor):
        return t.dtype, fp8sq.pack_fp8sq(t)
    if isinstance(t, nint8zero.Nint8ZeroTensor):
        return nint8zero.NINT8_ZERO_DTYPE, nint8zero.pack_nint8_zero(t)
    if isinstance(t, npq0.Npq0Tensor):
        return t.variant.label, npq0.pack_npq0(t)
    if isinstance(t, nvq1.Nvq1Tensor):
        return t.variant.label, nvq1.pack_nvq1(t)
    if isinstance(t, nepq.NepqTensor):
        return nepq.NEPQ_DTYPE, nepq.pack_nepq(t)
    if isinstance(t, nint.NintTensor):
        return nint.NINT_DTYPE, nint.pack_nint(t)
    if isinstance(t, (nvq.NvqTensor, nvq.NvqJscTensor)):
        return nvq.NVQ_DTYPE, nvq.pack_nvq(t)
    if isinstance(t, mfe.MfeTensor):
        return MFE_DTYPE, mfe.pack_mfe(t, pack_tensor)
    if isinstance(t, np.ndarray):
        return pack_dense(t)
    raise TypeError(f"unsupported tensor type {type(t)!r}")


def unpack_tensor(dtype: str, blob):
    if dtype == ASSET_DTYPE:
        return bytes(blob)
    if dtype in (mx.MXFP4_DTYPE, mx.MXFP8_DTYPE):
        return mx.unpack_mx(dtype, blob)
    if dtype == nint8zero.NINT8_ZERO_DTYPE:
        return nint8zero.unpack_nint8_zero(blob)
    if dtype in npq0.VARIANTS:
        return npq0.unpack_npq0(blob)
    if dtype in nvq1.DTYPES:
        return nvq1.unpack_nvq1(blob)
    if dtype == nepq.NEPQ_DTYPE:
        return nepq.unpack_nepq(blob)
    dtype = canonical_dtype(dtype)
    if dtype == MFE_DTYPE:
        return mfe.unpack_mfe(blob, unpack_tensor)
    if dtype == mxfp4sq.MXFP4_SQ_DTYPE:
        return mxfp4sq.unpack_mxfp4sq(blob)
    if dtype in (fp8sq.FP8_128SQ_DTYPE, fp8sq.MXFP8_SQ_DTYPE):
        return fp8sq.unpack_fp8sq(dtype, blob)
    if dtype == nint.NINT_DTYPE:
        return nint.unpack_nint(blob)
    if dtype == nvq.NVQ_DTYPE:
        return nvq.unpack_nvq(blob)
    if dtype in DENSE_DTYPES:
        return unpack_dense(dtype, blob)
    raise ValueError(f"unsupported tensor dtype {dtype!r}")


def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<I", len(b)) + b


def _header_bytes(header: FileHeader, records: list[tuple[str, str, int]]) -> bytes:
    version = int(header.version)
    if header.extra and version < 2:
        version = 2
    parts = [MFQ_MAGIC, struct.pack("<I", version), _s(header.model_arch)]
    if version >= 2:
        parts.append(struct.pack("<I", len(header.extra)))
        for k, v in header.extra.items():
            parts += [_s(str(k)), _s(json.dumps(v))]
    parts.append(struct.pack("<I", len(records)))
    for name, dtype, nbytes in records:
        parts += [_s(name), _s(dtype), struct.pack("<Q", nbytes)]
    return b"".join(parts)


def save(path, header: FileHeader, tensors: Mapping[str, Any]) -> None:
    """Write one ``.mfq`` file holding ``tensors`` (in mapping order)."""
    packed = {name: pack_tensor(t) for name, t in tensors.items()}
    records = [(name, dt, len(blob)) for name, (dt, blob) in packed.items()]
    tmp = f"{path}.tmp-{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(_header_bytes(header, records))
        for _dt, blob in packed.values():
            f.write(blob)
    os.replace(tmp, path)


def save_sharded(path, header: FileHeader, tensors: Mapping[str, Any], max_bytes: int | None,
                 max_tensors: int | None = None) -> list[Path]:
    """Write ``tensors`` as ``stem-00001-of-0000N.mfq`` files of at most ``max_bytes`` of blobs each (a tensor is never
    split; one larger than the limit gets a shard of its own).  Every shard carries the header; the asset records go to
    the first.  ``max_tensors`` also limits the records per shard.  Returns the shard paths; ``open_mfq`` on any of them
    opens the whole checkpoint."""
    p = Path(path)
    stem = p.name[: -len(".mfq")] if p.name.endswith(".mfq") else p.name
    packed = {name: pack_tensor(t) for name, t in tensors.items()}
    groups: list[list[str]] = [[]]
    size = 0
    for name, (_dt, blob) in packed.items():
        if groups[-1] and ((max_bytes and size + len(blob) > max_bytes) or (max_tensors and len(groups[-1]) >= max_tensors)):
            groups.append([])
            size = 0
        groups[-1].append(name)
        size += len(blob)
    paths = [p.with_name(f"{stem}-{i:05d}-of-{len(groups):05d}.mfq") for i in range(1, len(groups) + 1)]
    for shard, names in zip(paths, groups):
        records = [(n, packed[n][0], len(packed[n][1])) for n in names]
        tmp = f"{shard}.tmp-{os.getpid()}"
        with open(tmp, "wb") as f:
            f.write(_header_bytes(header, records))
            for n in names:
                f.write(packed[n][1])
        os.replace(tmp, shard)
    return paths


def write_streaming(path, header: FileHeader, items: list[tuple[str, str, int]], blob_iter) -> None:
    """Write a file whose blobs are produced lazily (``blob_iter`` yields bytes per record).

    ``items`` carries ``(name, dtype, nbytes)`` up front so the table can be written
    first; used by the quantize flow, which never holds more than one tensor.
    """
    tmp = f"{path}.tmp-{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(_header_bytes(header, items))
        for (name, _dt, nbytes), blob in zip(items, blob_iter, strict=True):
            if len(blob) != nbytes:
                raise ValueError(f"blob of {name!r} has {len(blob)} bytes, table says {nbytes}")
            f.write(blob)
    os.replace(tmp, path)


class _Cursor:
    def __init__(self, buf) -> None:
        self.buf, self.off = buf, 0

    def u32(self) -> int:
        (v,) = struct.unpack_from("<I", self.buf, self.off)
        self.off += 4
        return v

    def u64(self) -> int:
        (v,) = struct.unpack_from("<Q", self.buf, self.off)
        self.off += 8
        return v

    def text(self) -> str:
        n = self.u32()
        if self.off + n > len(self.buf):
            raise ValueError("truncated .mfq header string")
        s = bytes(self.buf[self.off : self.off + n]).decode("utf-8")
        self.off += n
        return s


def _parse_header(buf, file_index: int) -> tuple[FileHeader, list[TensorRecord]]:
    if bytes(buf[:4]) != MFQ_MAGIC:
        raise ValueError("not an MFQ1 file")
    c = _Cursor(buf)
    c.off = 4
    version = c.u32()
    arch = c.text()
    extra: dict[str, Any] = {}
    if version >= 2:
        for _ in range(c.u32()):
            k = c.text()
            extra[k] = json.loads(c.text())
    table = []
    for _ in range(c.u32()):
        name, dtype = c.text(), c.text()
        table.append((name, dtype, c.u64()))
    off = c.off
    records = []
    for name, dtype, nbytes in table:
        records.append(TensorRecord(name, dtype, off, nbytes, file_index))
        off += nbytes
    if off > len(buf):
        raise ValueError("truncated .mfq file: blobs run past the end")
    return FileHeader(version, arch, extra), records


def shard_paths(path) -> list[Path]:
    """All files of the checkpoint that ``path`` belongs to, in shard order."""
    p = Path(path)
    m = _SHARD_RE.match(p.name)
    if not m:
        return [p]
    count = int(m["count"])
    return [p.with_name(f"{m['stem']}-{i:05d}-of-{count:05d}.mfq") for i in range(1, count + 1)]


class MfqStore(Mapping[str, Any]):
    """Lazy, memory-mapped view of a (possibly sharded) checkpoint."""

    def __init__(self, path) -> None:
        self.paths = shard_paths(path)
        self._files, self._maps = [], []
        self.records: dict[str, TensorRecord] = {}
        self.header = FileHeader()
        for i, p in enumerate(self.paths):
            f = open(p, "rb")
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._files.append(f)
            self._maps.append(m)
            header, records = _parse_header(m, i)
            if i == 0:
                self.header = header
            for r in records:
                if r.name in self.records:
                    raise ValueError(f"tensor {r.name!r} appears in more than one shard")
                self.records[r.name] = r

    def raw(self, name: str) -> memoryview:
        r = self.records[name]
        return memoryview(self._maps[r.file_index])[r.offset : r.offset + r.nbytes]

    def dtype(self, name: str) -> str:
        return canonical_dtype(self.records[name].dtype)

    def __getitem__(self, name: str):
        r = self.records[name]
        return unpack_tensor(r.dtype, self.raw(name))

    def __iter__(self) -> Iterator[str]:
        return iter(self.records)

    def __len__(self) -> int:
        return len(self.records)

    def assets(self) -> dict[str, bytes]:
        return {n[len(ASSET_PREFIX):]: bytes(self.raw(n)) for n in self.records if n.startswith(ASSET_PREFIX)}

    def close(self) -> None:
        for m in self._maps:
            try:
                m.close()
            except BufferError:  # a caller still holds a view
                pass
        for f in self._files:
            f.close()
        self._maps, self._files = [], []

    def __enter__(self) -> "MfqStore":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def open_mfq(path) -> MfqStore:
    return MfqStore(path)


def load(path) -> tuple[FileHeader, dict[str, Any]]:
    with MfqStore(path) as store:
        return store.header, {name: store[name] for name in store}

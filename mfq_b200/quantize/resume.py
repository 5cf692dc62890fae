"""Resumable quantization: every finished tensor is parked as a validated blob beside the output.

A long quantization (hours for a large MoE) that dies at tensor 700 of 900 should not start over.  While it runs,
each quantized tensor is written atomically (temporary name, then rename) to ``<output>.tmp/<digest>.blob``; a later
run with ``--resume`` takes a tensor from there instead of quantizing it again, but only if the blob still matches:

* its key -- SHA-256 over the tensor name, shape, the source values and the label of the plan for that tensor (format,
  expert assignment, importance digest) -- equals the key computed now, so a changed source or a changed plan
  re-quantizes;
* its payload has the recorded length and SHA-256, so a blob cut short by the crash is ignored.

The directory goes away after a successful run unless ``--keep-temp`` is given.  Reference behaviour:
``--resume`` / ``--resume-completed`` / ``--keep-temp`` of ``mfq/tools/quantize_hf_to_mfq.py`` (validated temporary
blobs) and the atomic statistics caches described in ``docs/quantization/alphaq.md:60-67``.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
from pathlib import Path

import numpy as np

from ..formats.container import pack_tensor, unpack_tensor

_MAGIC = b"MFQRESUME1\n"


class ResumeStore:
    def __init__(self, directory, resume: bool = False, keep: bool = False) -> None:
        self.dir, self.keep = Path(directory), keep
        if self.dir.exists() and not resume:
            shutil.rmtree(self.dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.reused: list[str] = []
        self.written: list[str] = []

    @staticmethod
    def key(name: str, array: np.ndarray, label: str) -> str:
        h = hashlib.sha256()
        h.update(json.dumps([name, list(array.shape), str(array.dtype), label]).encode())
        h.update(np.ascontiguousarray(array).view(np.uint8).data)
        return h.hexdigest()

    def _path(self, name: str) -> Path:
        return self.dir / (hashlib.sha1(name.encode()).hexdigest() + ".blob")

    def get(self, name: str, key: str):
        """The parked tensor, or None when there is none, it belongs to another source / plan, or it is damaged."""
        p = self._path(name)
        try:
            with open(p, "rb") as f:
                if f.read(len(_MAGIC)) != _MAGIC:
                    return None
                meta = json.loads(f.readline())
                blob = f.read()
        except (OSError, ValueError):
            return None
        if meta.get("name") != name or meta.get("key") != key or len(blob) != meta.get("nbytes"):
            return None
        if hashlib.sha256(blob).hexdigest() != meta.get("sha256"):
            return None
        self.reused.append(name)
        return unpack_tensor(meta["dtype"], blob)

    def put(self, name: str, key: str, tensor) -> None:
        dtype, blob = pack_tensor(tensor)
        blob = bytes(blob)
        meta = {"name": name, "key": key, "dtype": dtype, "nbytes": len(blob), "sha256": hashlib.sha256(blob).hexdigest()}
        p = self._path(name)
        tmp = p.with_suffix(".part")
        with open(tmp, "wb") as f:
            f.write(_MAGIC)
            f.write(json.dumps(meta).encode() + b"\n")
            f.write(blob)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, p)
        self.written.append(name)

    def finish(self) -> None:
        """Called after the output file is complete."""
        if not self.keep:
            shutil.rmtree(self.dir, ignore_errors=True)

"""Builds the in-tree CUDA library ``_mfq_b200_kernels.so`` for sm_100a with plain ``nvcc``.

The kernels expose a C ABI (raw pointers + ``cudaStream_t``) and are loaded with ``ctypes``, so the
library has no dependency on PyTorch headers, compiles in seconds and cross-compiles on a machine
without a GPU.  ``python -m mfq_b200.ops.build`` rebuilds it; ``build(force=False)`` is incremental.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_PATH = HERE / "_mfq_b200_kernels.so"
OBJ_DIR = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for header in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(header.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: Path, force: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    digest = _digest(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, ""
    cmd = [nvcc_path(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stderr}")
    stamp.write_text(digest)
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link the shared library.  Returns its path."""
    OBJ_DIR.mkdir(exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile_one(s, force), srcs))
    objs = [str(o) for o, _ in results]
    log = "".join(text for _, text in results)
    if log:
        (OBJ_DIR / "ptxas.log").write_text(log)
    rebuilt = any(text for _, text in results)
    if rebuilt or not LIB_PATH.exists():
        cmd = [nvcc_path(), "--shared", "-o", str(LIB_PATH), *objs]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stderr}")
    if verbose and log:
        print(log, file=sys.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))

"""Builds the host runtime library (``_mfq_core.so``) from ``native/src`` with g++ (no CUDA dependency)."""

from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "src"
LIB = HERE / "_mfq_core.so"


def sources() -> list[Path]:
    return sorted(SRC.glob("*.cpp"))


def stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(SRC.glob("*.cpp")) + list(SRC.glob("*.h")))
    return newest > LIB.stat().st_mtime


def build(force: bool = False) -> Path:
    if not force and not stale():
        return LIB
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-Wall", "-Wextra", "-o", str(LIB)] + [str(p) for p in sources()]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))

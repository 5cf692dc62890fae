"""Runs the benchmark's metric on the unmodified reference, through the reference's own runtime."""

from __future__ import annotations


def run(args) -> dict:
    return {"impl": "reference", "unavailable": "reference native runtime (cpp_runtime, CUDA) is not built into baseline/_ref yet; only its Python package is installed"}

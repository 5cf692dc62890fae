"""TurboQuant-style KV codec on the CPU: rotate, normalise, scalar-quantize (2 .. 8 bits per value, halves allowed).

A head vector is multiplied by a fixed randomised Hadamard rotation (sign flips + fast Walsh-Hadamard transform), which
spreads its energy so that every rotated coordinate is close to Gaussian; the vector's norm is kept as an f16 and each
coordinate of the normalised vector goes through the Lloyd-Max quantizer of the standard normal at ``b`` bits.  A
fractional setting such as 2.5 bits gives the first half of the coordinates ``ceil(b)`` bits and the second half
``floor(b)``.  This is the host-side codec for KV snapshots that leave the GPU (session snapshots, offloaded blocks); the
GPU cache itself stays FP8 pages.  Levels and validation follow the reference's setting (``bits`` in 2, 2.5, 3, 3.5, 4,
6, 8; ``tests/test_kv_quantization_settings.py``); the packed layout is this repo's own, not the reference's CUDA one
(``cpp_runtime/backends/cuda/kernels/kv_quantization.cu``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

import numpy as np

LEVELS = (2, 2.5, 3, 3.5, 4, 6, 8)


@lru_cache(maxsize=None)
def lloyd_max_gaussian(bits: int) -> tuple[np.ndarray, np.ndarray]:
    """(centroids [2^b], decision thresholds [2^b - 1]) of the mean-square-optimal quantizer of N(0, 1)."""
    n = 1 << bits
    x = np.linspace(-6.0, 6.0, 48001)
    pdf = np.exp(-0.5 * x * x)
    c = np.quantile(np.random.default_rng(0).standard_normal(200_000), (np.arange(n) + 0.5) / n)
    for _ in range(200):
        t = 0.5 * (c[1:] + c[:-1])
        idx = np.searchsorted(t, x)
        mass = np.bincount(idx, weights=pdf, minlength=n)
        mean = np.bincount(idx, weights=pdf * x, minlength=n) / np.maximum(mass, 1e-300)
        if np.max(np.abs(mean - c)) < 1e-7:
            c = mean
            break
        c = mean
    return c.astype(np.float32), (0.5 * (c[1:] + c[:-1])).astype(np.float32)


def _fwht(x: np.ndarray) -> np.ndarray:
    """Fast Walsh-Hadamard transform along the last axis (length a power of two), orthonormal."""
    n = x.shape[-1]
    y = x.reshape(-1, n).astype(np.float32, copy=True)
    h = 1
    while h < n:
        y = y.reshape(-1, n // (2 * h), 2, h)
        a, b = y[:, :, 0, :].copy(), y[:, :, 1, :].copy()
        y[:, :, 0, :], y[:, :, 1, :] = a + b, a - b
        h *= 2
    return (y.reshape(x.shape) / math.sqrt(n)).astype(np.float32)


@lru_cache(maxsize=None)
def _signs(dim: int, seed: int) -> np.ndarray:
    return np.where(np.random.default_rng(seed).integers(0, 2, dim) == 1, 1.0, -1.0).astype(np.float32)


@dataclass
class TurboBlock:
    dim: int
    bits: float
    seed: int
    norms: np.ndarray  # [n] float16
    hi: np.ndarray  # packed codes of the first half (ceil(bits) bits each), uint8
    lo: np.ndarray  # packed codes of the second half (floor(bits) bits each), uint8
    rows: int

    @property
    def nbytes(self) -> int:
        return self.norms.nbytes + self.hi.nbytes + self.lo.nbytes


def _pack(codes: np.ndarray, bits: int) -> np.ndarray:
    planes = ((codes.reshape(-1, 1).astype(np.uint16) >> np.arange(bits, dtype=np.uint16)) & 1).astype(np.uint8)
    return np.packbits(planes.reshape(-1), bitorder="little")


def _unpack(buf: np.ndarray, count: int, bits: int) -> np.ndarray:
    planes = np.unpackbits(buf, bitorder="little")[: count * bits].reshape(count, bits).astype(np.uint16)
    return (planes << np.arange(bits, dtype=np.uint16)).sum(1).astype(np.uint16)


def validate_bits(bits) -> float:
    if isinstance(bits, bool) or not isinstance(bits, (int, float)) or bits != bits or bits not in LEVELS:
        raise ValueError(f"KV quantization level must be one of {LEVELS}, got {bits!r}")
    return float(bits)


def encode(x: np.ndarray, bits: float = 4, seed: int = 0) -> TurboBlock:
    """``x [rows, dim]`` (dim a power of two) -> :class:`TurboBlock`."""
    bits = validate_bits(bits)
    x = np.asarray(x, dtype=np.float32)
    rows, dim = x.shape
    if dim & (dim - 1):
        raise ValueError("the head dimension must be a power of two")
    norms = np.linalg.norm(x, axis=1).astype(np.float16)
    unit = x / np.maximum(norms.astype(np.float32), 1e-12)[:, None]
    z = _fwht(unit * _signs(dim, seed)) * math.sqrt(dim)  # coordinates ~ N(0, 1)
    half = dim // 2
    b_hi, b_lo = math.ceil(bits), math.floor(bits)
    hi = np.searchsorted(lloyd_max_gaussian(b_hi)[1], z[:, :half]).astype(np.uint16)
    lo = np.searchsorted(lloyd_max_gaussian(b_lo)[1], z[:, half:]).astype(np.uint16)
    return TurboBlock(dim, bits, seed, norms, _pack(hi, b_hi), _pack(lo, b_lo), rows)


def decode(blk: TurboBlock) -> np.ndarray:
    half = blk.dim // 2
    b_hi, b_lo = math.ceil(blk.bits), math.floor(blk.bits)
    z = np.empty((blk.rows, blk.dim), dtype=np.float32)
    z[:, :half] = lloyd_max_gaussian(b_hi)[0][_unpack(blk.hi, blk.rows * half, b_hi)].reshape(blk.rows, half)
    z[:, half:] = lloyd_max_gaussian(b_lo)[0][_unpack(blk.lo, blk.rows * half, b_lo)].reshape(blk.rows, half)
    unit = _fwht(z / math.sqrt(blk.dim)) * _signs(blk.dim, blk.seed)  # the rotation is its own inverse up to the signs
    return unit * blk.norms.astype(np.float32)[:, None]

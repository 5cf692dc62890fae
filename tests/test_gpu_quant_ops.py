"""Quantizer-side CUDA kernels against their PyTorch formulation."""

import numpy as np
import pytest
import torch

from gpu_common import require_gpu_lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("vec,codes,vectors", [(8, 256, 1000), (8, 4096, 20000), (4, 512, 7777), (8, 1024, 257)])
def test_fused_nvq_assignment_matches_the_cost_matrix_argmin(vec, codes, vectors):
    require_gpu_lib()
    from mfq_b200.quantize.nvq import _assign, assign_fused
    g = torch.Generator(device="cuda").manual_seed(vec * codes)
    table = torch.randint(0, 8, (codes, vec), generator=g, device="cuda").float() * 2 + 1  # odd lattice-like entries
    x = torch.randn((vectors, vec), generator=g, device="cuda").abs() * 6
    w = torch.rand((vectors, vec), generator=g, device="cuda") + 0.05
    s = torch.rand(vectors, generator=g, device="cuda") + 0.3
    got = assign_fused(x, w, table, s)
    cross, quad = (w * x) @ table.T, w @ (table * table).T
    want = _assign(cross, quad, s)
    cost = s[:, None] ** 2 * quad - 2 * s[:, None] * cross
    c_got, c_want = cost.gather(1, got[:, None])[:, 0], cost.gather(1, want[:, None])[:, 0]
    # equal up to ties / last-bit differences of the two summation orders
    assert float((c_got - c_want).abs().max()) <= 1e-3 * float(c_want.abs().max())
    assert float((got == want).float().mean()) > 0.99


def test_nvq_quantizer_on_the_gpu_matches_the_cpu_quality():
    require_gpu_lib()
    from mfq_b200 import formats as F
    from mfq_b200.formats.nvq import NvqSpec
    from mfq_b200.quantize.nvq import quantize_nvq
    w = np.random.default_rng(0).standard_normal((64, 528)).astype(np.float32)  # 22 groups of 24
    spec = NvqSpec("e8_1024")
    cpu = quantize_nvq(w, spec, device="cpu")
    gpu = quantize_nvq(w, spec, device="cuda")
    e_cpu = float(((np.asarray(F.dequantize(cpu)) - w) ** 2).sum())
    e_gpu = float(((np.asarray(F.dequantize(gpu)) - w) ** 2).sum())
    assert e_gpu <= e_cpu * 1.02


def test_jsc_quantizer_on_the_gpu_matches_the_cpu_quality():
    """The state / entry assignment of the NVQ-JSC quantizer through the fused nearest-codeword kernel (one launch per
    state, no vectors-by-entries matrices) reaches the error of the matrix form on the CPU; the MXFP4-SQ and NEPQ
    encoders are device-agnostic torch / NumPy and need no kernel."""
    require_gpu_lib()
    from mfq_b200 import formats as F
    from mfq_b200.quantize.nvq_jsc import quantize_nvq_jsc
    w = (np.random.default_rng(1).standard_t(df=6, size=(96, 240)) * 0.03).astype(np.float32)
    for grid, banks in (("e8_256", 2), ("d4_256", 1)):
        cpu = quantize_nvq_jsc(w, grid, banks=banks, iterations=2, device="cpu")
        gpu = quantize_nvq_jsc(w, grid, banks=banks, iterations=2, device="cuda")
        e_cpu = float(((np.asarray(F.dequantize(cpu)) - w) ** 2).sum())
        e_gpu = float(((np.asarray(F.dequantize(gpu)) - w) ** 2).sum())
        assert e_gpu <= e_cpu * 1.03, (grid, e_cpu, e_gpu)
        assert F.pack_tensor(F.unpack_tensor(*F.pack_tensor(gpu)))[1] == F.pack_tensor(gpu)[1]

"""4-bit group-quantized GEMM with in-pipeline decode against ``x @ dequantize(W)^T`` (fp32 reference)."""

import numpy as np
import pytest
import torch

from mfq_b200.ops import w4
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def _weight(n, k, gs, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, (n, k)).astype(np.uint8)
    s = (rng.random((n, k // gs)) * 0.01 + 0.002).astype(np.float32)
    b = (rng.random((n, k // gs)) * 0.08).astype(np.float32)
    return w4.repack(codes, s, b, gs)


@pytest.mark.parametrize("m,n,k,gs,splits", [(1, 256, 256, 32, 1), (16, 200, 1024, 32, 3), (64, 384, 4096, 16, 4), (128, 128, 192, 24, 1),
                                             (300, 520, 2048, 64, 2), (33, 4096, 4096, 32, None)])
def test_w4_gemm_matches_reference(m, n, k, gs, splits):
    require_gpu_lib()
    w = _weight(n, k, gs, m + n)
    g = torch.Generator(device="cuda").manual_seed(k)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    res = torch.randn((m, n), generator=g, device="cuda").to(torch.bfloat16)
    wd = w.to("cuda")
    got = w4.w4_gemm(x, wd, residual=res, splits=splits)
    check_status()
    want = x.float() @ w4.dequantize(w).cuda().T + res.float()
    assert_close(got.float(), want, rel=1e-2, what="w4 gemm")
    again = w4.w4_gemm(x, wd, residual=res, splits=splits)  # split-K reduction is order-independent: bit-identical
    assert torch.equal(got, again)


def test_w4_from_nint_checkpoint_tensor():
    require_gpu_lib()
    from mfq_b200.formats import nint
    from mfq_b200.quantize.nint import quantize_nint
    rng = np.random.default_rng(5)
    wf = (rng.standard_normal((256, 768)) * 0.05).astype(np.float32)
    t = quantize_nint(wf, nint.NintSpec(bits=4, groupsize=24, sub_bits=6))
    w = w4.from_nint(t)
    x = torch.randn((8, 768), device="cuda").to(torch.bfloat16)
    got = w4.w4_gemm(x, w.to("cuda"))
    check_status()
    want = x.float() @ torch.from_numpy(nint.dequantize_nint(t)).cuda().T  # the checkpoint's own reconstruction
    # the kernel keeps each group's (scale, minimum) in bf16: the minimum is ~8 code steps, so its 2^-9 rounding alone
    # moves a weight by a few percent of a step; outputs near zero see that as about 1 % of the output rms
    assert_close(got.float(), want, rel=6e-2, what="w4 gemm vs NINT dequantization")
    assert w.bits_per_weight < 5.5


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (48, 300, 2048), (200, 512, 4096)])
def test_mxfp4_kind_matches_checkpoint_dequantization(m, n, k):
    """MXFP4 tensors run through the same pipeline with the E2M1 table decode: exact weights, bf16 x bf16 products."""
    require_gpu_lib()
    from mfq_b200 import formats as F
    from mfq_b200.quantize.mxfp4 import quantize_mxfp4
    rng = np.random.default_rng(m)
    t = quantize_mxfp4((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    w = w4.from_mxfp4(t)
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    got = w4.w4_gemm(x, w.to("cuda"))
    check_status()
    want = x.float() @ torch.from_numpy(F.dequantize(t)).cuda().T
    assert_close(got.float(), want, rel=1e-2, what="mxfp4 gemm")

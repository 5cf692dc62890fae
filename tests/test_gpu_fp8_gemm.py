"""tcgen05 block-scaled FP8 GEMM against the fp32 dequantize-then-matmul reference."""

import pytest
import torch

from mfq_b200 import ops
from mfq_b200.ops import reference as ref
from mfq_b200.quantize.fp8_block import quantize_fp8_block_torch
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def make(m, n, k, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    xq, xs = ref.quant_rows(x)
    wq, ws = quantize_fp8_block_torch(w)
    return xq, xs, wq, ws


@pytest.mark.parametrize("m,n,k,splits", [
    (1, 128, 128, 1), (16, 256, 512, 1), (5, 384, 1024, 1), (40, 512, 512, 1), (64, 1024, 2048, 1),
    (128, 256, 1024, 1), (300, 640, 1536, 1), (512, 1024, 4096, 1),
    (1, 256, 2048, 4), (33, 384, 4096, 8), (64, 512, 14336, 7), (130, 256, 1024, 2),
    # up to 8 splits meet in distributed shared memory (one cluster per tile), more go through the global scratch buffer
    (20, 320, 2048, 3), (64, 256, 4096, 16), (100, 4096, 4096, 4), (64, 6144, 4096, 3), (7, 384, 1536, 6),
])
def test_fp8_gemm_matches_reference(m, n, k, splits):
    require_gpu_lib()
    xq, xs, wq, ws = make(m, n, k, seed=m + n)
    got = ops.fp8_gemm(xq, xs, wq, ws, splits=splits)
    check_status()
    assert_close(got, ref.fp8_gemm(xq, xs, wq, ws), what=f"gemm {m}x{n}x{k} s{splits}")


def test_fp8_gemm_residual_inplace_and_repeatable():
    require_gpu_lib()
    xq, xs, wq, ws = make(48, 512, 2048)
    res = torch.randn((48, 512), device="cuda").to(torch.bfloat16)
    want = ref.fp8_gemm(xq, xs, wq, ws, residual=res)
    h = res.clone()
    ops.fp8_gemm(xq, xs, wq, ws, residual=h, out=h, splits=1)
    h2 = res.clone()
    ops.fp8_gemm(xq, xs, wq, ws, residual=h2, out=h2, splits=4)
    check_status()
    assert_close(h, want, what="residual")
    assert_close(h2, want, what="residual split-K")
    a = ops.fp8_gemm(xq, xs, wq, ws, splits=4)
    b = ops.fp8_gemm(xq, xs, wq, ws, splits=4)
    assert torch.equal(a, b), "split-K reduction must be deterministic"
    counters = ops.Workspace.get(xq.device).counters
    assert int(counters.abs().sum().item()) == 0, "tile counters must return to zero"


def test_fp8_gemm_all_token_tiles():
    require_gpu_lib()
    xq, xs, wq, ws = make(16, 256, 1024)
    want = ref.fp8_gemm(xq, xs, wq, ws)
    for tile in (16, 32, 64, 128):
        assert_close(ops.fp8_gemm(xq, xs, wq, ws, token_tile=tile, splits=1), want, what=f"tile {tile}")
    check_status()


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (1, 4096, 4096), (4, 6144, 2048), (8, 2048, 14336), (9, 272, 1024),
                                   (16, 1040, 512), (2, 151936, 256), (17, 768, 4096), (32, 1024, 512), (47, 512, 1024),
                                   (64, 768, 4096), (64, 16, 128)])
def test_weight_streaming_gemv_matches_reference(m, n, k):
    """Rows <= 16 (and up to 64 rows on small matrices) without explicit tiling take the mma.sync weight-streaming
    kernel (residual add in place included)."""
    require_gpu_lib()
    assert ops.kernels.use_gemv(m, n, k)
    xq, xs, wq, ws = make(m, n, k, seed=3 * m + n)
    res = torch.randn((m, n), device="cuda").to(torch.bfloat16)
    want = ref.fp8_gemm(xq, xs, wq, ws, residual=res)
    got = ops.fp8_gemm(xq, xs, wq, ws, residual=res)
    check_status()
    assert_close(got, want, what=f"gemv {m}x{n}x{k}")
    # the tcgen05 GEMM agrees on the same problem
    assert_close(ops.fp8_gemm(xq, xs, wq, ws, residual=res, splits=1), want, what="gemm on the gemv shape")
    h = res.clone()
    ops.fp8_gemm(xq, xs, wq, ws, residual=h, out=h)
    assert_close(h, want, what="gemv residual in place")


@pytest.mark.parametrize("tile", [128, 256])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (300, 512, 1024), (1024, 768, 2048)])
def test_fp8_gemm_on_sm_pairs_matches_reference(m, n, k, tile):
    """The two-SM kernel (a CTA pair per 256 weight rows, tokens shared through the tensor core's peer read)."""
    require_gpu_lib()
    xq, xs, wq, ws = make(m, n, k, seed=m + n + tile)
    res = torch.randn((m, n), device="cuda").to(torch.bfloat16)
    got = ops.fp8_gemm(xq, xs, wq, ws, pair=tile, residual=res)
    check_status()
    assert_close(got, ref.fp8_gemm(xq, xs, wq, ws, residual=res), what=f"pair gemm {m}x{n}x{k} tile {tile}")
    again = ops.fp8_gemm(xq, xs, wq, ws, pair=tile, residual=res)
    assert torch.equal(got, again)


@pytest.mark.parametrize("m,n,k", [(1, 6144, 4096), (3, 256, 2048), (4, 4096, 8192), (2, 512, 1024), (1, 4096, 14336)])
def test_gemv_with_folded_activation_preparation_is_bit_identical(m, n, k):
    """RMSNorm + quantization, plain quantization and SwiGLU + quantization done inside the product kernel give the bits
    of the standalone kernels followed by the weight-streaming product (the sum of squares replays the norm kernel's
    summation tree), with and without an in-place residual."""
    require_gpu_lib()
    g = torch.Generator(device="cuda").manual_seed(m * 31 + n)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    wq, ws = quantize_fp8_block_torch(w)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, generator=g, device="cuda")).to(torch.bfloat16)
    res = torch.randn((m, n), generator=g, device="cuda").to(torch.bfloat16)
    # norm
    xq, xs, _, _ = ops.rmsnorm_quant(x, nw, 1e-5)
    want = ops.fp8_gemm(xq, xs, wq, ws)
    got = ops.fp8_gemv_act(x, wq, ws, ops.ACT_NORM, norm_w=nw, eps=1e-5)
    assert torch.equal(got, want), float((got.float() - want.float()).abs().max())
    # plain, residual added in place
    xq, xs = ops.quant_rows(x)
    want = ops.fp8_gemm(xq, xs, wq, ws, residual=res)
    h = res.clone()
    ops.fp8_gemv_act(x, wq, ws, ops.ACT_PLAIN, residual=h, out=h)
    assert torch.equal(h, want)
    # SwiGLU
    gu = torch.randn((m, 2 * k), generator=g, device="cuda").to(torch.bfloat16)
    hq, hs = ops.silu_mul_quant(gu)
    want = ops.fp8_gemm(hq, hs, wq, ws, residual=res)
    got = ops.fp8_gemv_act(gu, wq, ws, ops.ACT_SWIGLU, residual=res)
    assert torch.equal(got, want)
    check_status()
    assert_close(got, ref.fp8_gemm(*ref.silu_mul_quant(gu), wq, ws, residual=res), what="against the fp32 restatement")

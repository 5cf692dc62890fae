"""The allocation-free GEMM entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory at the point where they need the GEMM (inside a stream
capture, inside a serving loop that must not synchronize, or because they gave the library a fixed memory budget),
so ``mfq_fp8_gemm_noalloc`` keeps its split-K scratch in a device array inside the library.  This test checks that
it gives the same answer as the regular entry point and as the fp32 reference, twice in a row (the second call
reuses the scratch the first one left behind), and that the status word reads back clean.
"""

import ctypes as C

import pytest
import torch

from gpu_common import assert_close, require_gpu_lib

pytestmark = pytest.mark.gpu


def _noalloc(lib, w, ws, x, xs, out, residual, tile, splits):
    fn = lib.mfq_fp8_gemm_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int] * 5 + [C.c_void_p]
    m, k = x.shape
    return fn(w.data_ptr(), ws.data_ptr(), x.data_ptr(), xs.data_ptr(), out.data_ptr(),
              None if residual is None else residual.data_ptr(), m, w.shape[0], k, tile, splits,
              torch.cuda.current_stream().cuda_stream)


def test_noalloc_entry_matches_regular_entry_twice():
    lib = require_gpu_lib()
    from mfq_b200 import ops
    from mfq_b200.ops import reference as ref
    from mfq_b200.quantize.fp8_block import quantize_fp8_block_torch
    g = torch.Generator(device="cuda").manual_seed(11)
    for call, (m, n, k, tile, splits) in enumerate([(48, 512, 2048, 64, 4), (16, 384, 4096, 16, 8)]):
        x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        res = torch.randn((m, n), generator=g, device="cuda").to(torch.bfloat16)
        xq, xs = ref.quant_rows(x)
        wq, wsc = quantize_fp8_block_torch(w)
        want = ops.fp8_gemm(xq, xs, wq, wsc, residual=res, splits=splits, token_tile=tile)
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = _noalloc(lib, wq, wsc, xq, xs, got, res, tile, splits)
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert_close(got, want, rel=2e-2, what=f"no-alloc call {call}")
        assert torch.equal(got, want), "same kernel, same split order: results must be identical"
        exact = ref.fp8_gemm(xq.cpu(), xs.cpu(), wq.cpu(), wsc.cpu(), residual=res.cpu())
        assert_close(got.cpu(), exact, rel=2e-2, what=f"no-alloc call {call} vs fp32 reference")
        status = C.c_int(-1)
        st = lib.mfq_fp8_gemm_noalloc_status
        st.restype, st.argtypes = C.c_int, [C.POINTER(C.c_int), C.c_void_p]
        assert st(C.byref(status), torch.cuda.current_stream().cuda_stream) == 0 and status.value == 0


def test_noalloc_entry_rejects_oversized_problem():
    lib = require_gpu_lib()
    x = torch.zeros((128, 128), device="cuda", dtype=torch.uint8)
    s = torch.ones(1024, device="cuda")
    # 8192 x 1024 output tiles cannot fit 4096 counters; nothing is launched for a rejected call
    fn = lib.mfq_fp8_gemm_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int] * 5 + [C.c_void_p]
    rc = fn(x.data_ptr(), s.data_ptr(), x.data_ptr(), s.data_ptr(), x.data_ptr(), None, 16384, 1 << 20, 128, 16, 1, None)
    assert rc == -20
    rc = fn(x.data_ptr(), s.data_ptr(), x.data_ptr(), s.data_ptr(), x.data_ptr(), None, 16, 128, 100, 16, 1, None)
    assert rc == -1

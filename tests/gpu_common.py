"""Shared helpers of the GPU tests: they require the in-tree CUDA library and fail loudly without it."""

import pytest
import torch


def require_gpu_lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mfq_b200.ops.lib import LIB_PATH, lib
    assert LIB_PATH.exists(), "the CUDA library must be built in-tree before GPU tests run"
    return lib()


def assert_close(actual, expected, rel=2e-2, what=""):
    a, e = actual.float(), expected.float()
    err = (a - e).abs().max().item()
    ref = e.abs().max().item() + 1e-6
    assert err <= rel * ref, f"{what}: max abs err {err:.4g} vs ref magnitude {ref:.4g}"


def check_status():
    from mfq_b200.ops import Workspace
    torch.cuda.synchronize()
    Workspace.get(torch.device("cuda", torch.cuda.current_device())).check()

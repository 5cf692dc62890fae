"""Shared helpers of the GPU tests: they require the in-tree CUDA library and fail loudly without it."""

import pytest
import torch


def require_gpu_lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mfq_b200.ops.lib import LIB_PATH, lib
    assert LIB_PATH.exists(), "the CUDA library must be built in-tree before GPU tests run"
    return lib()


def assert_close(actual, expected, rel=2e-2, what="", outliers=1e-3):
    """Two criteria.  (1) The largest error stays within ``rel`` of the largest reference magnitude.  (2) Element by
    element, ``|err| <= rel * (|ref| + rms(ref) / 4)`` for all but a fraction ``outliers`` of the elements, so that an
    error confined to the small outputs (invisible to the first criterion) fails too."""
    a, e = actual.float(), expected.float()
    diff = (a - e).abs()
    err = diff.max().item()
    ref = e.abs().max().item() + 1e-6
    assert err <= rel * ref, f"{what}: max abs err {err:.4g} vs ref magnitude {ref:.4g}"
    rms = e.pow(2).mean().sqrt().item() + 1e-12
    bad = (diff > rel * (e.abs() + 0.25 * rms)).float().mean().item()
    assert bad <= outliers, f"{what}: {bad:.3%} of the elements are off by more than {rel:g} x (|ref| + rms/4), rms {rms:.4g}"


def check_status():
    from mfq_b200.ops import Workspace
    torch.cuda.synchronize()
    Workspace.get(torch.device("cuda", torch.cuda.current_device())).check()

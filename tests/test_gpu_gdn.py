"""Gated DeltaNet kernels against the fp32 torch restatement: decode, prefill-length runs, verify windows."""

import pytest
import torch

from mfq_b200.ops import gdn
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def _problem(b, L, hk, hv, slots, seed):
    g = torch.Generator().manual_seed(seed)
    dk = dv = 128
    c = 2 * hk * dk + hv * dv
    n = b * L
    t = dict(
        x=(torch.randn((n, c), generator=g) * 0.8).to(torch.bfloat16),
        z=torch.randn((n, hv * dv), generator=g).to(torch.bfloat16),
        a=torch.randn((n, hv), generator=g).to(torch.bfloat16),
        b=torch.randn((n, hv), generator=g).to(torch.bfloat16),
        w=torch.randn((c, 4), generator=g) * 0.5,
        A_log=torch.randn(hv, generator=g) * 0.5,
        dt_bias=torch.randn(hv, generator=g) * 0.5,
        norm_w=1 + 0.1 * torch.randn(dv, generator=g),
        conv_state=torch.randn((slots, 3, c), generator=g).to(torch.bfloat16).float(),
        state=torch.randn((slots, hv, dk, dv), generator=g) * 0.1,
        slot=torch.randperm(slots, generator=g)[:b].to(torch.int32),
    )
    return t, c


def _run(t, dev, L, hk, hv, ckpt=False):
    d = {k: v.clone().to(dev) for k, v in t.items()}
    b = d["slot"].numel()
    cck = torch.zeros((b, L, 3, d["x"].shape[1]), device=dev) if ckpt else None
    sck = torch.zeros((b, L, hv, 128, 128), device=dev) if ckpt else None
    qkv = gdn.conv(d["x"], d["conv_state"], d["w"], d["slot"], L, conv_ckpt=cck)
    conv_out = qkv.clone()  # long rows normalise q and k inside qkv
    y = gdn.recurrent(qkv, d["z"], d["a"], d["b"], d["A_log"], d["dt_bias"], d["norm_w"], d["state"], d["slot"], L, hk, hv,
                      ckpt=sck)
    return conv_out, y, d, cck, sck


@pytest.mark.parametrize("b,L,hk,hv", [(5, 1, 2, 4), (1, 67, 2, 2), (3, 4, 1, 2), (1, 9, 1, 2), (3, 300, 2, 4), (1, 1024, 1, 1),
                                       (1, 64, 1, 2), (2, 2048, 2, 4)])
def test_gdn_matches_reference(b, L, hk, hv):
    require_gpu_lib()
    t, _ = _problem(b, L, hk, hv, slots=b + 2, seed=b * 10 + L)
    t["slot"][b // 2] = -1 if b > 2 else t["slot"][b // 2]  # a masked row must leave its state untouched
    qg, yg, dg, _, _ = _run(t, "cuda", L, hk, hv)
    qc, yc, dc, _, _ = _run(t, "cpu", L, hk, hv)
    check_status()
    live = (t["slot"] >= 0).repeat_interleave(L)
    assert_close(qg.cpu()[live], qc[live], rel=1e-4, what="conv")
    assert_close(yg.float().cpu()[live], yc.float()[live], rel=2e-2, what="gdn output")
    assert_close(dg["state"].cpu(), dc["state"], rel=1e-3, what="state")
    assert_close(dg["conv_state"].cpu(), dc["conv_state"], rel=1e-6, what="conv state")


def test_gdn_token_serial_prefill_still_matches(monkeypatch):
    """Rows shorter than a chunk keep the token-serial long-row kernels; force them for a longer row too."""
    require_gpu_lib()
    monkeypatch.setattr(gdn, "CHUNKED_MIN_TOKENS", 1 << 30)
    t, _ = _problem(2, 150, 2, 4, slots=3, seed=5)
    _, yg, dg, _, _ = _run(t, "cuda", 150, 2, 4)
    _, yc, dc, _, _ = _run(t, "cpu", 150, 2, 4)
    check_status()
    assert_close(yg.float().cpu(), yc.float(), rel=2e-2, what="gdn output")
    assert_close(dg["state"].cpu(), dc["state"], rel=1e-3, what="state")


def test_gdn_chunked_prefill_equals_token_serial_kernels(monkeypatch):
    """The chunked scan runs its products in tf32; against the fp32 token-serial kernels on the same device the raw
    state differs by about a tf32 step (2^-11) of its largest entry."""
    require_gpu_lib()
    t, _ = _problem(1, 1000, 2, 4, slots=2, seed=9)
    _, y_chunk, d_chunk, _, _ = _run(t, "cuda", 1000, 2, 4)
    monkeypatch.setattr(gdn, "CHUNKED_MIN_TOKENS", 1 << 30)
    _, y_serial, d_serial, _, _ = _run(t, "cuda", 1000, 2, 4)
    check_status()
    assert_close(d_chunk["state"].cpu(), d_serial["state"].cpu(), rel=1.5e-3, what="state")
    assert_close(y_chunk.float().cpu(), y_serial.float().cpu(), rel=1e-2, what="gdn output")


def test_gdn_verify_window_checkpoints_and_select():
    require_gpu_lib()
    b, L, hk, hv = 3, 4, 1, 2
    t, _ = _problem(b, L, hk, hv, slots=4, seed=3)
    _, yg, dg, cck, sck = _run(t, "cuda", L, hk, hv, ckpt=True)
    # the window leaves the live state alone
    assert torch.equal(dg["state"].cpu(), t["state"]) and torch.equal(dg["conv_state"].cpu(), t["conv_state"])
    keep = torch.tensor([0, 3, 2], dtype=torch.int32, device="cuda")
    gdn.select(sck, cck, dg["state"], dg["conv_state"], dg["slot"], keep)
    check_status()
    # oracle: run only the kept prefix of every row, one row at a time
    for r in range(b):
        n = int(keep[r]) + 1
        sub = {k: v.clone() for k, v in t.items()}
        rows = slice(r * L, r * L + n)
        for name in ("x", "z", "a", "b"):
            sub[name] = t[name][rows]
        sub["slot"] = t["slot"][r : r + 1]
        _, yc, dc, _, _ = _run(sub, "cpu", n, hk, hv)
        s = int(t["slot"][r])
        assert_close(dg["state"][s].cpu(), dc["state"][s], rel=1e-3, what=f"state row {r}")
        assert_close(dg["conv_state"][s].cpu(), dc["conv_state"][s], rel=1e-6, what=f"conv state row {r}")
        assert_close(yg[r * L : r * L + n].float().cpu(), yc.float(), rel=2e-2, what=f"y row {r}")

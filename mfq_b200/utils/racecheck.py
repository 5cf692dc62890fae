"""Race and stale-scratch detection without a sanitizer: run an operator twice, poison what it must not depend on.

A kernel that reads scratch memory before writing it, that depends on the order in which its CTAs happen to run, or that
leaves a counter or flag behind gives different bits from one launch to the next once its scratch holds garbage.  The
check here exploits that: between two runs of ``fn`` every scratch tensor of the device workspace (split-K partials,
attention partials) is filled with a NaN bit pattern -- counters and the status word, which kernels are required to
leave at zero, are verified to BE zero instead -- and the outputs of the two runs are compared bit for bit.  It needs no
tool that instruments the process and costs two launches, so it runs inside the ordinary GPU test suite.

Reference: the reference has no in-tree sanitizer configuration either; its design notes record ad-hoc
``compute-sanitizer`` runs and byte-exact fused-vs-unfused replays (``bench/cuda_format_comparison/*.md``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class RaceReport:
    name: str
    runs: int
    bit_identical: bool
    finite: bool
    counters_clean: bool
    status: int
    mismatches: list[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return self.bit_identical and self.finite and self.counters_clean and self.status == 0


def poison_workspace(ws) -> None:
    """Fill the scratch tensors with a quiet-NaN pattern (fp32 0x7FC0DEAD; as bytes it is garbage for every type)."""
    for t in (ws.splitk, ws.attn_acc, ws.attn_ml):
        flat = t.view(torch.uint8).reshape(-1)
        n = flat.numel() // 4 * 4
        flat[:n].view(torch.int32).fill_(0x7FC0DEAD)


def _outputs(result) -> list[torch.Tensor]:
    if isinstance(result, torch.Tensor):
        return [result]
    if isinstance(result, (list, tuple)):
        return [t for r in result for t in _outputs(r)]
    return []


def check(name: str, fn, *, runs: int = 3, device=None) -> RaceReport:
    """``fn()`` -> tensor or nested tuple of tensors.  Runs it ``runs`` times with the workspace poisoned before each run
    and compares every output bit for bit with the first run's."""
    from ..ops import Workspace
    dev = torch.device(device or "cuda")
    ws = Workspace.get(dev)
    first: list[torch.Tensor] | None = None
    report = RaceReport(name, runs, True, True, True, 0)
    for r in range(runs):
        poison_workspace(ws)
        out = [t.detach().clone() for t in _outputs(fn())]
        torch.cuda.synchronize(dev)
        if int(ws.counters.abs().max().item()) != 0:
            report.counters_clean = False
            ws.counters.zero_()
        for i, t in enumerate(out):
            if t.is_floating_point() and not bool(torch.isfinite(t.float()).all()):
                report.finite = False
                report.mismatches.append(f"run {r}: output {i} holds non-finite values")
        if first is None:
            first = out
            continue
        for i, (a, b) in enumerate(zip(first, out)):
            same = a.shape == b.shape and torch.equal(a.view(torch.uint8) if a.element_size() == 1 else a.contiguous().view(-1).view(torch.uint8),
                                                      b.view(torch.uint8) if b.element_size() == 1 else b.contiguous().view(-1).view(torch.uint8))
            if not same:
                report.bit_identical = False
                report.mismatches.append(f"run {r}: output {i} differs from run 0")
    report.status = int(ws.status[0].item())
    return report

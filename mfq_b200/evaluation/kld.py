"""Quality metrics of a quantized model against a baseline: KL divergence and top-1 agreement.

Same definitions as the reference evaluator (``cpp_runtime/backends/cuda/eval/kl.cpp:216-220,316-326``):
``KLD = mean_t sum_v p_base(v) * (log p_base(v) - log q(v))`` over the scored positions, its reverse, and the share
of positions where both models rank the same token first.  :func:`teacher_forced_report` scores a quantized model
on the token sequence the baseline generated (prompt, then greedy continuation), position by position.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class KldReport:
    kld: float
    reverse_kld: float
    top1_agreement: float
    positions: int
    max_kld: float

    def as_dict(self) -> dict:
        return {"kld": self.kld, "reverse_kld": self.reverse_kld, "same_top": self.top1_agreement,
                "positions": self.positions, "max_kld": self.max_kld}


def compare_logits(base: torch.Tensor, test: torch.Tensor) -> KldReport:
    """``base`` / ``test``: ``[positions, vocab]`` logits."""
    lp = torch.log_softmax(base.double(), -1)
    lq = torch.log_softmax(test.double(), -1)
    kl = (lp.exp() * (lp - lq)).sum(-1)
    rkl = (lq.exp() * (lq - lp)).sum(-1)
    same = (lp.argmax(-1) == lq.argmax(-1)).double().mean()
    return KldReport(float(kl.mean()), float(rkl.mean()), float(same), int(kl.numel()), float(kl.max()))


def teacher_forced_report(base_model, test_model, prompt: torch.Tensor, new_tokens: int) -> tuple[KldReport, torch.Tensor]:
    """Greedy-decode ``new_tokens`` with ``base_model``; feed the same tokens to ``test_model``; compare the logits of
    every position from the last prompt token on.  Models expose ``reset()`` and ``forward(ids) -> logits``."""
    base_model.reset()
    test_model.reset()
    lb = [base_model.forward(prompt)]
    lt = [test_model.forward(prompt)]
    nxt = lb[0][-1].argmax().reshape(1)
    generated = [int(nxt)]
    for _ in range(new_tokens - 1):
        lb.append(base_model.forward(nxt))
        lt.append(test_model.forward(nxt))
        nxt = lb[-1][-1].argmax().reshape(1)
        generated.append(int(nxt))
    base = torch.cat([lb[0][-1:]] + lb[1:])
    test = torch.cat([lt[0][-1:]] + lt[1:])
    all_base = torch.cat([lb[0]] + lb[1:])
    all_test = torch.cat([lt[0]] + lt[1:])
    report = compare_logits(all_base, all_test)
    report_decode = compare_logits(base, test)
    report.max_kld = max(report.max_kld, report_decode.max_kld)
    return report, torch.tensor(generated)

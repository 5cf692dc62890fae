"""Speculative-decoding policies: verification rules and the adaptive depth controller."""

import torch

from mfq_b200.engine.mtp_policy import DepthController, verify_greedy, verify_stochastic


def test_greedy_verification():
    assert verify_greedy(torch.tensor([5, 6, 7]), torch.tensor([5, 6, 9, 1])) == (2, 9)
    assert verify_greedy(torch.tensor([5, 6, 7]), torch.tensor([5, 6, 7, 1])) == (3, 1)
    assert verify_greedy(torch.tensor([4]), torch.tensor([5, 2])) == (0, 5)


def test_stochastic_verification_preserves_the_target_distribution():
    """One draft position: whatever the draft distribution is, the first emitted token follows the target's."""
    g = torch.Generator().manual_seed(0)
    p = torch.tensor([0.5, 0.3, 0.15, 0.05])
    q = torch.tensor([0.1, 0.1, 0.2, 0.6])  # a poor draft
    target = torch.stack([p, torch.tensor([0.25, 0.25, 0.25, 0.25])])
    counts, accepted, n = torch.zeros(4), 0, 20000
    for _ in range(n):
        x = int(torch.multinomial(q, 1, generator=g))
        k, nxt = verify_stochastic(torch.tensor([x]), q[None], target, generator=g)
        accepted += k
        counts[x if k == 1 else nxt] += 1
    assert torch.allclose(counts / n, p, atol=0.015)
    assert abs(accepted / n - float(torch.minimum(p, q).sum())) < 0.015  # acceptance rate = overlap of the distributions
    # a perfect draft is always accepted
    assert verify_stochastic(torch.tensor([1]), p[None], target, generator=g)[0] == 1


def _run(ctrl, true_accept, cost, cycles, seed=0):
    g = torch.Generator().manual_seed(seed)
    tokens = ms = 0.0
    for _ in range(cycles):
        d = ctrl.next_depth()
        acc = 0
        while acc < d and float(torch.rand(1, generator=g)) < true_accept[acc]:
            acc += 1
        ctrl.observe(d, acc, cost[d])
        tokens += acc + 1
        ms += cost[d]
    return tokens / ms


def test_depth_controller_finds_the_profitable_depth_and_parks_when_there_is_none():
    cost = [10.0, 11.0, 12.0, 13.0]
    good = DepthController(3)
    rate = _run(good, [0.9, 0.85, 0.8], cost, 600)
    assert good.next_depth() == 3 and not good.parked and rate > 1.6 / 10.0  # well above plain decode's 0.1 tokens/ms
    assert abs(good.acceptance[0] - 0.9) < 0.15
    mid = DepthController(3)
    _run(mid, [0.8, 0.1, 0.1], cost, 600)
    assert mid.next_depth() in (1, 2) and not mid.parked  # deeper drafts are rejected: a shallow chain wins
    bad = DepthController(3)
    _run(bad, [0.05, 0.05, 0.05], cost, 600)
    assert bad.parked and bad.next_depth() == 0
    # parked controllers keep probing, so a draft head that becomes useful again is noticed
    _run(bad, [0.9, 0.9, 0.9], cost, 1500, seed=1)
    assert not bad.parked and bad.next_depth() == 3

"""Tiny random-init MoE LM with per-expert-projection NINT4 / NVQ3 / MXFP4 experts: container round trip and
KLD / top-1 agreement of the quantized model against the bf16 model (CPU)."""

import torch

from mfq_b200 import formats as F
from mfq_b200.evaluation.kld import compare_logits, teacher_forced_report
from mfq_b200.models.moe_lm import MoeConfig, MoeLM, dequantize_checkpoint, init_weights, quantize_moe_checkpoint


def test_quantized_tiny_moe_tracks_bf16(tmp_path):
    cfg = MoeConfig()
    w = init_weights(cfg, seed=0)
    q = quantize_moe_checkpoint(w, "NINT4,NVQ3,MXFP4", seed=20260908)
    # every routed projection mixes all three families, balanced over the 8 experts
    gate = q["model.block.0.mlp.experts.gate.weight"]
    assert sorted(len(p.expert_ids) for p in gate.pools) == [2, 3, 3]
    assert {type(p.tensor).__name__ for p in gate.pools} == {"NintTensor", "NvqTensor", "MxTensor"}
    path = tmp_path / "tiny_moe.mfq"
    F.save(path, F.FileHeader(model_arch="tiny_moe", extra={"config": cfg.__dict__}), q)
    _, loaded = F.load(path)
    wq = dequantize_checkpoint(loaded)
    assert set(wq) == set(w)
    prompt = torch.randint(0, cfg.vocab_size, (64,), generator=torch.Generator().manual_seed(1))
    report, generated = teacher_forced_report(MoeLM(cfg, w), MoeLM(cfg, wq), prompt, 32)
    assert generated.numel() == 32 and report.positions == 64 + 31
    assert 0 <= report.kld < 0.05, report
    assert report.top1_agreement > 0.7, report


def test_kld_definition():
    a = torch.randn(10, 50)
    r = compare_logits(a, a)
    assert abs(r.kld) < 1e-12 and r.top1_agreement == 1.0
    b = a + 0.5 * torch.randn(10, 50)
    r2 = compare_logits(a, b)
    assert r2.kld > 0 and r2.reverse_kld > 0

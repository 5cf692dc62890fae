"""Tiny FP8 Llama end to end on the GPU: kernels vs the CPU reference path, graphs vs eager."""

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights, StepBuffers
from gpu_common import check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def to_device(w: LlamaWeights, dev):
    import copy
    import dataclasses
    w2 = copy.deepcopy(w)

    def mv(o):
        if torch.is_tensor(o):
            return o.to(dev)
        if dataclasses.is_dataclass(o):
            for f in dataclasses.fields(o):
                setattr(o, f.name, mv(getattr(o, f.name)))
            return o
        if isinstance(o, list):
            return [mv(x) for x in o]
        return o
    return mv(w2)


def test_tiny_llama_gpu_matches_cpu_reference():
    require_gpu_lib()
    cfg = LlamaConfig.tiny()
    w_cpu = LlamaWeights.random_init(cfg, "cpu", seed=1, std=0.05)
    w_gpu = to_device(w_cpu, "cuda")
    prompts = [torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(3)),
               torch.randint(0, cfg.vocab_size, (64,), generator=torch.Generator().manual_seed(4))]
    e_cpu = LLMEngine(LlamaModel(cfg, w_cpu), max_batch=2, max_seq_len=128, device="cpu")
    e_gpu = LLMEngine(LlamaModel(cfg, w_gpu), max_batch=2, max_seq_len=128, device="cuda", use_graphs=False)
    # logits of a prefill must agree closely
    for eng in (e_cpu, e_gpu):
        eng.row_seq = {}
    outs = []
    for eng in (e_cpu, e_gpu):
        dev = eng.device
        eng.cache.assign(0, 0, 64)
        eng.cache.allocator.owned.setdefault(0, eng.cache.allocator.owned[0])
        step = StepBuffers(input_ids=prompts[1].to(dev, torch.int32), positions=torch.arange(64, dtype=torch.int32, device=dev),
                           slots=eng.cache.slots(0, 0, 64).to(dev), cu_seqlens=[0, 64])
        outs.append(eng.model.forward(step, eng.cache, prefill=True).float().cpu())
        eng.cache.release(0)
    check_status()
    err = (outs[0] - outs[1]).abs().max().item()
    scale = outs[0].abs().max().item()
    assert err < 0.12 * scale, f"prefill logits differ: {err} vs {scale}"
    agree = (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean().item()
    assert agree > 0.9


def test_graph_decode_matches_eager():
    require_gpu_lib()
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cuda", seed=2, std=0.05)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (20, 45, 31)]
    a = LLMEngine(LlamaModel(cfg, w), max_batch=4, max_seq_len=128, use_graphs=False).generate(prompts, 12)
    b = LLMEngine(LlamaModel(cfg, w), max_batch=4, max_seq_len=128, use_graphs=True).generate(prompts, 12)
    assert torch.equal(a.tokens, b.tokens)
    check_status()

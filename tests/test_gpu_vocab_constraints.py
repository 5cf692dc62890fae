"""Token constraints on the GPU engine: the constrained graph variant masks the logits like the eager step does."""

import pytest
import torch

from mfq_b200 import native
from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.engine.scheduler import SamplingParams
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
from mfq_b200.server.tokenizer import ByteTokenizer
from gpu_common import require_gpu_lib

pytestmark = pytest.mark.gpu


def test_constrained_decode_graph_matches_eager_and_stays_in_the_grammar():
    require_gpu_lib()
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cuda", seed=7)
    tok = ByteTokenizer(cfg.vocab_size)
    fmt = SamplingParams(max_tokens=48, stop_token_ids=tok.stop_ids, response_format={"type": "json_object"})
    prompt = tok.encode("Reply in JSON.")
    outs = []
    for graphs in (True, False):
        eng = LLMEngine(LlamaModel(cfg, w), max_batch=4, max_seq_len=128, use_graphs=graphs)
        eng.set_token_bytes(lambda: tok.token_bytes(cfg.vocab_size), tok.stop_ids)
        free = eng.prefill(1, prompt, SamplingParams(max_tokens=8))  # an unconstrained neighbour in the same batch
        eng.grow(1, len(prompt) + 48)  # pages for every token the loop below may write
        seq = [eng.prefill(0, prompt, fmt)]
        eng.grow(0, len(prompt) + 48)
        neighbour = [free]
        for _ in range(40):
            if eng.row_constraint[0].finished:
                break
            step = eng.decode([0, 1])
            seq.append(step[0])
            neighbour.append(step[1])
        outs.append((seq, neighbour))
        text = bytes(t - 3 for t in seq if 3 <= t < 259)
        state = native.JsonState(eng._constraint_vocab, need_object=True)
        assert state.feed(text), text
        # the neighbour decodes as if alone: a row's tokens depend on the batch bucket (which fixes the kernels and
        # their summation order), not on what the other rows of the bucket hold
        alone = LLMEngine(LlamaModel(cfg, w), max_batch=4, max_seq_len=128, use_graphs=graphs)
        ref = [alone.prefill(1, prompt, SamplingParams(max_tokens=8))]
        alone.grow(1, len(prompt) + 48)
        for _ in range(len(neighbour) - 1):
            ref.append(alone.decode([1])[1])
        assert ref == neighbour
    assert outs[0] == outs[1]

"""Child process of the tensor-parallel GPU test: launched by torch.distributed.run, one rank per GPU."""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from mfq_b200.engine.llm_engine import LLMEngine  # noqa: E402
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights, StepBuffers  # noqa: E402
from mfq_b200.ops import Workspace  # noqa: E402
from mfq_b200.parallel.tensor_parallel import NcclTensorParallel, TensorParallel  # noqa: E402


def prefill_logits(model, engine, prompt, dev):
    n = prompt.numel()
    engine.cache.assign(0, 10_000, n)
    step = StepBuffers(input_ids=prompt.to(dev, torch.int32), positions=torch.arange(n, dtype=torch.int32, device=dev),
                       slots=engine.cache.slots(10_000, 0, n).to(dev), cu_seqlens=[0, n])
    out = model.forward(step, engine.cache, prefill=True).float()
    engine.cache.release(10_000)
    return out


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig.tiny()
    result = {"world": world}
    prompt = torch.randint(0, cfg.vocab_size, (48,), generator=torch.Generator().manual_seed(7))

    tp = TensorParallel(dist.group.WORLD, dev)
    w = LlamaWeights.random_init(cfg, dev, seed=3, std=0.05, tp_rank=rank, tp_size=world)
    model = LlamaModel(cfg, w, collective=tp)
    engine = LLMEngine(model, max_batch=4, max_seq_len=128)
    fused = prefill_logits(model, engine, prompt, dev)

    base_model = LlamaModel(cfg, w, collective=NcclTensorParallel(dist.group.WORLD, dev))
    base_engine = LLMEngine(base_model, max_batch=4, max_seq_len=128, use_graphs=False)
    nccl = prefill_logits(base_model, base_engine, prompt, dev)
    result["fused_vs_nccl_max_err"] = float((fused - nccl).abs().max())
    result["logit_scale"] = float(nccl.abs().max())

    w1 = LlamaWeights.random_init(cfg, dev, seed=3, std=0.05)
    m1 = LlamaModel(cfg, w1)
    e1 = LLMEngine(m1, max_batch=4, max_seq_len=128, use_graphs=False)
    single = prefill_logits(m1, e1, prompt, dev)
    result["tp_vs_single_max_err"] = float((fused - single).abs().max())
    result["tp_vs_single_top1"] = float((fused.argmax(-1) == single.argmax(-1)).float().mean())

    # graph decode: every rank must sample the same tokens
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (20, 33, 41)]
    toks = engine.generate(prompts, 10).tokens.to(dev)
    gathered = [torch.empty_like(toks) for _ in range(world)]
    dist.all_gather(gathered, toks)
    result["ranks_agree"] = all(torch.equal(g, gathered[0]) for g in gathered)
    eager = LLMEngine(LlamaModel(cfg, w, collective=tp), max_batch=4, max_seq_len=128, use_graphs=False)
    result["graph_equals_eager"] = bool(torch.equal(eager.generate(prompts, 10).tokens.to(dev), toks))
    # fused GEMM -> reduce-scatter and all-gather -> GEMM against unfused references
    from mfq_b200.models.llama import Fp8Linear
    from mfq_b200.ops import reference as ref
    g = torch.Generator(device=dev).manual_seed(11)  # same values on every rank
    m_tok, n_out, k_full = 256 * world, 384, 512 * world
    x_full = torch.randn((m_tok, k_full), generator=g, device=dev).to(torch.bfloat16)
    w_full = (torch.randn((n_out, k_full), generator=g, device=dev) * 0.05).to(torch.bfloat16)
    ks = k_full // world
    xq, xs = ref.quant_rows(x_full[:, rank * ks:(rank + 1) * ks])
    lin = Fp8Linear.from_float(w_full[:, rank * ks:(rank + 1) * ks].contiguous())
    partial = ref.fp8_gemm(xq, xs, lin.q, lin.scale).float()
    dist.all_reduce(partial)
    res = torch.randn((m_tok, n_out), generator=g, device=dev).to(torch.bfloat16)
    rows = slice(rank * m_tok // world, (rank + 1) * m_tok // world)
    for it in range(3):
        got = tp.gemm_reduce_scatter(lin, xq, xs, res[rows].contiguous(), token_tile=128)
        tp.barrier()
    want = (partial[rows] + res[rows].float())
    result["rs_max_err"] = float((got.float() - want).abs().max() / want.abs().max())
    w_col = Fp8Linear.from_float((torch.randn((256, 512), generator=g, device=dev) * 0.05).to(torch.bfloat16))
    xa = torch.randn((m_tok, 512), generator=g, device=dev).to(torch.bfloat16)
    xaq, xas = ref.quant_rows(xa)
    for it in range(3):
        got_ag = tp.allgather_gemm(w_col, xaq[rows].contiguous(), xas[rows].contiguous(), token_tile=128, push_ctas=4)
    want_ag = ref.fp8_gemm(xaq, xas, w_col.q, w_col.scale).float()
    result["ag_max_err"] = float((got_ag.float() - want_ag).abs().max() / want_ag.abs().max())
    torch.cuda.synchronize()
    Workspace.get(dev).check()

    # expert parallelism: routed experts split over the ranks, shared expert and attention tensor-parallel
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights, quantize_moe_checkpoint
    mcfg = MoeDecoderConfig.tiny()
    ck = quantize_moe_checkpoint(init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128,
                                                        shared_intermediate=128), seed=4, std=0.05), "NINT4,NVQ3,MXFP4")
    ep_model = MoeDecoderModel(mcfg, MoeWeights.from_tensors(mcfg, ck, dev, rank, world), collective=tp)
    ep_engine = LLMEngine(ep_model, max_batch=4, max_seq_len=128)
    ep_logits = prefill_logits(ep_model, ep_engine, prompt, dev)
    one_model = MoeDecoderModel(mcfg, MoeWeights.from_tensors(mcfg, ck, dev))
    one_logits = prefill_logits(one_model, LLMEngine(one_model, max_batch=4, max_seq_len=128, use_graphs=False), prompt, dev)
    result["ep_vs_single_max_err"] = float((ep_logits - one_logits).abs().max())
    result["ep_logit_scale"] = float(one_logits.abs().max())
    result["ep_vs_single_mean_err"] = float((ep_logits - one_logits).abs().mean())
    ep_toks = ep_engine.generate(prompts, 6).tokens.to(dev)
    gathered = [torch.empty_like(ep_toks) for _ in range(world)]
    dist.all_gather(gathered, ep_toks)
    result["ep_ranks_agree"] = all(torch.equal(g, gathered[0]) for g in gathered)
    torch.cuda.synchronize()
    Workspace.get(dev).check()
    dist.barrier()
    if rank == 0:
        print("TP_RESULT " + json.dumps(result), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

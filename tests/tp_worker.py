"""Child process of the tensor-parallel GPU test: launched by torch.distributed.run, one rank per GPU."""

import dataclasses
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
    if world > 2:  # enough heads / width for every rank to own whole 128-wide blocks
        cfg = dataclasses.replace(cfg, num_heads=8, num_kv_heads=8, intermediate_size=128 * world)
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
    # wide-batch row-parallel linear = reduce-scatter epilogue + all-gather of rows, repeated without barriers
    for it in range(3):
        h_full = res.clone()
        tp.row_parallel_linear(lin, xq, xs, h_full)
    want_full = partial + res.float()
    result["ar2_max_err"] = float((h_full.float() - want_full).abs().max() / want_full.abs().max())
    w_col = Fp8Linear.from_float((torch.randn((256, 512), generator=g, device=dev) * 0.05).to(torch.bfloat16))
    xa = torch.randn((m_tok, 512), generator=g, device=dev).to(torch.bfloat16)
    xaq, xas = ref.quant_rows(xa)
    for it in range(3):
        got_ag = tp.allgather_gemm(w_col, xaq[rows].contiguous(), xas[rows].contiguous(), token_tile=128, push_ctas=4)
    want_ag = ref.fp8_gemm(xaq, xas, w_col.q, w_col.scale).float()
    result["ag_max_err"] = float((got_ag.float() - want_ag).abs().max() / want_ag.abs().max())
    torch.cuda.synchronize()
    Workspace.get(dev).check()

    # fused all-reduce + residual + RMSNorm + FP8 quantization over peer memory, one-shot and two-shot, eager and replayed
    hid = 512
    st = tp.stream(hid)
    norm_w = (torch.rand(hid, generator=g, device=dev) + 0.5).to(torch.bfloat16)
    fr_h_exact, fr_q_err = True, 0.0
    for m_rows in (1, 24, 8 * world + 3, 200):
        for it in range(3):
            gr = torch.Generator(device=dev).manual_seed(100 * m_rows + 10 * it + rank)
            part = torch.randn((m_rows, hid), generator=gr, device=dev).to(torch.bfloat16)
            h0 = torch.randn((m_rows, hid), generator=torch.Generator(device=dev).manual_seed(7 + it), device=dev).to(torch.bfloat16)
            hbuf = st.h_rows(m_rows)
            hbuf.copy_(h0)
            tp.barrier()  # every rank's residual rows are in place before a peer may push into them
            st.partial_out(m_rows).copy_(part)
            _, xq_f, xs_f = st.reduce(m_rows, hbuf, norm_w, 1e-5)
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            total = torch.zeros((m_rows, hid), device=dev)
            for p_ in parts:
                total = total + p_.float()
            h_want = (total + h0.float()).to(torch.bfloat16)
            fr_h_exact = fr_h_exact and bool(torch.equal(hbuf, h_want))
            q_w, s_w, _, _ = ref.rmsnorm_quant(h_want, norm_w, 1e-5)
            got_x = xq_f.float() * xs_f[:, None]
            want_x = q_w.float() * s_w[:, None]
            fr_q_err = max(fr_q_err, float((got_x - want_x).abs().max() / want_x.abs().max()))
    result["fused_reduce_h_exact"], result["fused_reduce_q_err"] = fr_h_exact, fr_q_err
    torch.cuda.synchronize()
    Workspace.get(dev).check()

    # expert parallelism: routed experts split over the ranks, shared expert and attention tensor-parallel
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights, quantize_moe_checkpoint
    mcfg = MoeDecoderConfig.tiny()
    heads = dict(num_heads=8, num_kv_heads=8) if world > 2 else {}
    mcfg = dataclasses.replace(mcfg, **heads)
    ck = quantize_moe_checkpoint(init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128,
                                                        shared_intermediate=128, **heads), seed=4, std=0.05), "NINT4,NVQ3,MXFP4")
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
    # the same model with wide batches routed through the all-to-all (48 prompt tokens: 48 / world per rank)
    a2a_model = MoeDecoderModel(mcfg, MoeWeights.from_tensors(mcfg, ck, dev, rank, world), collective=tp)
    a2a_model.enable_expert_all_to_all(dist.group.WORLD, max_tokens=64, min_tokens=world)
    a2a_engine = LLMEngine(a2a_model, max_batch=4, max_seq_len=128, use_graphs=False)
    a2a_logits = prefill_logits(a2a_model, a2a_engine, prompt, dev)
    result["ep_a2a_vs_replicated_max_err"] = float((a2a_logits - ep_logits).abs().max())
    result["ep_a2a_vs_replicated_mean_err"] = float((a2a_logits - ep_logits).abs().mean())
    if world == 2:
        # hybrid model (Gated DeltaNet + gated attention + experts) with every head kind split over the two ranks
        from mfq_b200.models.hybrid import HybridConfig, HybridModel, HybridWeights, init_hybrid_weights
        hcfg = HybridConfig.tiny()
        ht = init_hybrid_weights(hcfg, seed=3, std=0.05)

        def hybrid_logits(model, graphs):
            eng = LLMEngine(model, max_batch=4, max_seq_len=128, use_graphs=graphs)
            n = prompt.numel()
            eng.cache.assign(0, 20_000, n)
            eng.rec_state.reset(0)
            step = StepBuffers(input_ids=prompt.to(dev, torch.int32), positions=torch.arange(n, dtype=torch.int32, device=dev),
                               slots=eng.cache.slots(20_000, 0, n).to(dev), cu_seqlens=[0, n], state_slots=eng.row_ids[:1])
            out = model.forward(step, eng.cache, prefill=True).float()
            eng.cache.release(20_000)
            return out, eng
        h_tp, h_eng = hybrid_logits(HybridModel(hcfg, HybridWeights.from_tensors(hcfg, ht, dev, rank, world), collective=tp), True)
        h_one, _ = hybrid_logits(HybridModel(hcfg, HybridWeights.from_tensors(hcfg, ht, dev)), False)
        result["hybrid_tp_cos"] = float(torch.nn.functional.cosine_similarity(h_tp.flatten(), h_one.flatten(), dim=0))
        result["hybrid_tp_row_cos"] = float(torch.nn.functional.cosine_similarity(h_tp, h_one, dim=1).median())
        h_toks = h_eng.generate(prompts, 6).tokens.to(dev)
        got = [torch.empty_like(h_toks) for _ in range(world)]
        dist.all_gather(got, h_toks)
        result["hybrid_ranks_agree"] = all(torch.equal(g, got[0]) for g in got)
    # token-sharded dispatch -> local experts -> combine through peer memory, against all experts on one GPU
    from mfq_b200.ops import moe as moe_ops
    from mfq_b200.ops import reference as ref
    from mfq_b200.parallel.expert_parallel import ExpertParallel, NcclExpertParallel
    from mfq_b200.quantize.fp8_block import quantize_fp8_block_torch
    g = torch.Generator(device=dev).manual_seed(11)  # same stream on every rank: identical global problem
    t_all, hh, inter, ne, kk = 96 * world, 512, 256, 8 * world, 4
    xa = torch.randn((t_all, hh), generator=g, device=dev).to(torch.bfloat16)
    gu_f = (torch.randn((ne, 2 * inter, hh), generator=g, device=dev) * 0.05).to(torch.bfloat16)
    dn_f = (torch.randn((ne, hh, inter), generator=g, device=dev) * 0.05).to(torch.bfloat16)
    gq, gs = (torch.stack(z) for z in zip(*[quantize_fp8_block_torch(m) for m in gu_f]))
    dq, ds = (torch.stack(z) for z in zip(*[quantize_fp8_block_torch(m) for m in dn_f]))
    ids_all = torch.stack([torch.randperm(ne, generator=g, device=dev)[:kk] for _ in range(t_all)]).to(torch.int32)
    wt_all = torch.rand((t_all, kk), generator=g, device=dev)
    base_all = torch.randn((t_all, hh), generator=g, device=dev).to(torch.bfloat16)
    xq_all, xs_all = ref.quant_rows(xa)
    want_all = moe_ops.moe_ffn_fp8(xq_all, xs_all, ids_all, wt_all, gq, gs, dq, ds, base=base_all).float()
    # uneven shards: rank r owns a different number of tokens
    cuts = [0] + [int(t_all * (r + 1) / world) - (7 if r + 1 < world else 0) for r in range(world)]
    lo, hi = cuts[rank], cuts[rank + 1]
    e_per = ne // world
    mine = slice(rank * e_per, (rank + 1) * e_per)
    ep = ExpertParallel(dist.group.WORLD, dev, num_experts=ne, top_k=kk, hidden=hh, max_tokens=128 * world)
    a2a_err = 0.0
    for _ in range(3):
        got = ep.moe_ffn(xq_all[lo:hi].contiguous(), xs_all[lo:hi].contiguous(), ids_all[lo:hi].contiguous(),
                         wt_all[lo:hi].contiguous(), gq[mine].contiguous(), gs[mine].contiguous(), dq[mine].contiguous(),
                         ds[mine].contiguous(), base=base_all[lo:hi].contiguous(), cap=max(b - a for a, b in zip(cuts, cuts[1:])))
        a2a_err = max(a2a_err, float((got.float() - want_all[lo:hi]).abs().max() / want_all.abs().max()))
    # library baseline moves the same rows
    nep = NcclExpertParallel(dist.group.WORLD, dev, num_experts=ne, top_k=kk, hidden=hh, max_tokens=0)
    rx, rs_, rids, rw, ctx = nep.dispatch(xq_all[lo:hi].contiguous(), xs_all[lo:hi].contiguous(), ids_all[lo:hi].contiguous(),
                                          wt_all[lo:hi].contiguous())
    y_tok = moe_ops.moe_ffn_fp8(rx, rs_, rids, rw, gq[mine].contiguous(), gs[mine].contiguous(), dq[mine].contiguous(),
                                ds[mine].contiguous(), e_lo=rank * e_per, base=None)
    got_n = nep.combine(y_tok, ctx, base=base_all[lo:hi])
    errs = torch.tensor([a2a_err, float((got_n.float() - want_all[lo:hi]).abs().max() / want_all.abs().max())], device=dev)
    dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    result["a2a_max_err"], result["a2a_nccl_max_err"] = float(errs[0]), float(errs[1])
    torch.cuda.synchronize()
    Workspace.get(dev).check()
    dist.barrier()
    if rank == 0:
        print("TP_RESULT " + json.dumps(result), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

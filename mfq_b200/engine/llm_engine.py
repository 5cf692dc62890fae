"""In-process generation engine: chunked prefill, CUDA-graph decode, greedy sampling.

The decode step is captured once per batch bucket.  Everything a step needs lives on the device: the sampled
token feeds the next step, positions / sequence lengths / KV slots are advanced by a kernel inside the graph,
so replaying the graph needs no host work and the host reads tokens back only when it wants them.  (The
reference replays its decode graph and then synchronizes on ``static_next.item()`` once per token,
``cpp_runtime/backends/cuda/engine/generation.cpp:304-339``.)
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..models.llama import LlamaModel, StepBuffers
from .kv_cache import PAGE_SIZE, PagedKVCache

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128)


@dataclass
class GenerationResult:
    tokens: torch.Tensor  # [B, new_tokens] int32 (cpu)
    prefill_ms: float
    decode_ms: float
    prompt_tokens: int
    new_tokens: int


class LLMEngine:
    def __init__(self, model: LlamaModel, *, max_batch: int = 64, max_seq_len: int = 8192, num_pages: int | None = None,
                 device=None, use_graphs: bool = True, prefill_chunk: int = 8192) -> None:
        self.model = model
        cfg = model.cfg
        self.device = torch.device(device) if device is not None else model.w.embed.device
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        self.prefill_chunk = prefill_chunk
        pages_per_seq = (max_seq_len + PAGE_SIZE - 1) // PAGE_SIZE
        if num_pages is None:
            num_pages = max_batch * pages_per_seq + 1
        self.cache = PagedKVCache(layers=cfg.num_layers, kv_heads=model.hk, head_dim=cfg.head_dim, num_pages=num_pages,
                                  max_seqs=max_batch, max_pages_per_seq=pages_per_seq, device=self.device)
        dev = self.device
        self.input_ids = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.seq_lens = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.slots = torch.full((max_batch,), -1, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.use_graphs = use_graphs and dev.type == "cuda"
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._next_seq_id = 0
        self.launches_per_step: dict[int, int] = {}

    # -- prefill -------------------------------------------------------------------------------------------------
    def prefill(self, row: int, token_ids: torch.Tensor) -> int:
        """Run the prompt of batch row ``row`` through the model; returns the first generated token id and leaves
        the row ready for decode (``seq_lens[row]`` = prompt length, ``sampled[row]`` = first token)."""
        dev = self.device
        n = int(token_ids.numel())
        seq_id = self._next_seq_id
        self._next_seq_id += 1
        self.row_seq = getattr(self, "row_seq", {})
        if row in self.row_seq:
            self.cache.release(self.row_seq[row])
        self.row_seq[row] = seq_id
        self.cache.assign(row, seq_id, min(self.max_seq_len, n + 1))
        ids = token_ids.to(dev, dtype=torch.int32, non_blocking=True)
        last = None
        for start in range(0, n, self.prefill_chunk):
            end = min(n, start + self.prefill_chunk)
            if start > 0:
                raise NotImplementedError("multi-chunk prefill needs attention over earlier pages")
            step = StepBuffers(
                input_ids=ids[start:end], positions=torch.arange(start, end, dtype=torch.int32, device=dev),
                slots=self.cache.slots(seq_id, start, end - start).to(dev), cu_seqlens=[0, end - start])
            rows = torch.tensor([end - start - 1], dtype=torch.int32, device=dev)
            logits = self.model.forward(step, self.cache, prefill=True, logits_rows=rows, gather_logits=False)
            last = logits
        tok = self.model.sample_greedy(last)
        self.sampled[row : row + 1] = tok
        self.seq_lens[row] = n
        return tok

    def grow(self, row: int, tokens: int) -> None:
        self.cache.assign(row, self.row_seq[row], min(self.max_seq_len, tokens))

    # -- decode --------------------------------------------------------------------------------------------------
    def _decode_body(self, b: int) -> None:
        dev = self.device
        if dev.type == "cuda":
            ops.decode_advance(self.sampled[:b], self.input_ids[:b], self.positions[:b], self.seq_lens[:b], self.slots[:b],
                               self.cache.block_table[:b], self.cache.page_size)
        else:
            self.input_ids[:b] = self.sampled[:b]
            pos = self.seq_lens[:b].clone()
            self.positions[:b] = pos
            pages = self.cache.block_table[:b].gather(1, (pos // self.cache.page_size).long()[:, None])[:, 0]
            self.slots[:b] = pages * self.cache.page_size + pos % self.cache.page_size
            self.seq_lens[:b] = pos + 1
        step = StepBuffers(input_ids=self.input_ids[:b], positions=self.positions[:b], slots=self.slots[:b],
                           block_table=self.cache.block_table[:b], seq_lens=self.seq_lens[:b])
        if dev.type == "cuda":
            from ..ops.kernels import attn_splits_for
            self.model.attn_splits = attn_splits_for(b, self.model.hk, self.max_seq_len)
        logits = self.model.forward(step, self.cache, prefill=False, gather_logits=False)
        self.model.sample_greedy(logits, out=self.sampled[:b])

    def decode_step(self, b: int) -> None:
        """Advance rows ``[0, b)`` by one token (result in ``self.sampled[:b]``, on the device)."""
        if not self.use_graphs:
            self._decode_body(b)
            return
        g = self.graphs.get(b)
        if g is None:
            ops.Workspace.get(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            saved = (self.seq_lens.clone(), self.sampled.clone())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode_body(b)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(g):
                self._decode_body(b)
            self.launches_per_step[b] = ops.launch_count() - before
            # warm-up and capture ran real steps: roll the sequence state back (the KV rows they wrote get rewritten)
            self.seq_lens.copy_(saved[0])
            self.sampled.copy_(saved[1])
            self.graphs[b] = g
        g.replay()

    def step_host(self, host_in: torch.Tensor, host_out: torch.Tensor) -> None:
        """One decode step driven from the host: ``host_in`` (pinned int32 ``[b]``, the tokens to feed) is copied
        to the device, the step runs, and the sampled ids land in ``host_out`` (pinned) before this returns."""
        b = host_in.numel()
        self.sampled[:b].copy_(host_in, non_blocking=True)
        self.decode_step(b)
        host_out.copy_(self.sampled[:b], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    # -- convenience ---------------------------------------------------------------------------------------------
    def generate(self, prompts: list[torch.Tensor], max_new_tokens: int) -> GenerationResult:
        """Static-batch greedy generation (all prompts prefilled, then decoded together)."""
        b = len(prompts)
        assert b <= self.max_batch
        cuda = self.device.type == "cuda"
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if cuda else None
        if cuda:
            ev[0].record()
        for row, p in enumerate(prompts):
            self.prefill(row, p)
            self.grow(row, int(p.numel()) + max_new_tokens + 1)
        if cuda:
            ev[1].record()
        out = torch.empty((b, max_new_tokens), dtype=torch.int32, device=self.device)
        out[:, 0] = self.sampled[:b]
        for t in range(1, max_new_tokens):
            self.decode_step(b)
            out[:, t] = self.sampled[:b]
        if cuda:
            ev[2].record()
            torch.cuda.synchronize()
            ops.Workspace.get(self.device).check()
        return GenerationResult(out.cpu(), ev[0].elapsed_time(ev[1]) if cuda else 0.0,
                                ev[1].elapsed_time(ev[2]) if cuda else 0.0, sum(int(p.numel()) for p in prompts),
                                b * max_new_tokens)

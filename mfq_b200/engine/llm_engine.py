"""In-process generation engine: prefill, CUDA-graph decode, greedy and stochastic sampling, row management.

The decode step is captured once per batch bucket.  Everything a step needs lives on the device: the sampled
token feeds the next step, positions / sequence lengths / KV slots are advanced by a kernel inside the graph,
rows that are not generating are masked by a device-side ``active`` vector, so replaying the graph needs no host
work and the host reads tokens back only when it wants them.  (The reference replays its decode graph and then
synchronizes on ``static_next.item()`` once per token, ``cpp_runtime/backends/cuda/engine/generation.cpp:304-339``;
its batch graphs are cached per row bucket {1,2,4,8,16,32}, ``runtime/batch_decode_graph.h:14-24``.)

The class also implements the backend protocol of :class:`~mfq_b200.engine.scheduler.ContinuousBatchScheduler`
(``prefill`` / ``decode`` / ``can_grow`` / ``release`` / capacity queries).
"""

from __future__ import annotations

import ctypes as C
import time
from dataclasses import dataclass

import torch

from .. import ops
from ..models.llama import LlamaModel, StepBuffers
from ..utils.profiler import scope
from .kv_cache import PAGE_SIZE, PagedKVCache

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
from ..config import current as _config, trace

_PROFILE_DECODE = _config().profile_decode  # one stderr line per decode call


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return n


@dataclass
class GenerationResult:
    tokens: torch.Tensor  # [B, new_tokens] int32 (cpu)
    prefill_ms: float
    decode_ms: float
    prompt_tokens: int
    new_tokens: int


class LLMEngine:
    def __init__(self, model: LlamaModel, *, max_batch: int = 64, max_seq_len: int = 8192, num_pages: int | None = None,
                 device=None, use_graphs: bool | None = None, mtp_draft_tokens: int = 0, prefill_chunk: int | None = None,
                 prefix_cache=None, prefix_salt: str = "", mtp_adaptive: bool = False, mtp_dynamic_depth: bool = False) -> None:
        """``mtp_draft_tokens`` (K, 0 = off): with a model that carries an MTP head, greedy rows decode by
        draft/verify cycles that confirm between 1 and K+1 tokens each (:meth:`mtp_step`).  ``mtp_dynamic_depth``: every
        cycle runs at the depth (1 .. K drafts) whose measured tokens per millisecond is best
        (:class:`~mfq_b200.engine.mtp_policy.CycleDepthController`); one graph per (bucket, depth, next depth)."""
        self.model = model
        # adaptive speculation: cycles only while they beat plain decoding (see engine/mtp_policy.ParkingController)
        self.mtp_controller = None
        if mtp_adaptive and mtp_draft_tokens:
            from .mtp_policy import ParkingController
            self.mtp_controller = ParkingController()
        use_graphs = _config().cuda_graphs if use_graphs is None else use_graphs
        prefill_chunk = _config().prefill_chunk if prefill_chunk is None else prefill_chunk
        self.prefill_chunk = prefill_chunk  # prompts longer than this are prefilled in chunks that attend to the cached past
        # content-addressed KV blocks (mfq_b200.native.PrefixCache): a prompt whose leading 256-token blocks are cached
        # gets their pages restored instead of recomputed.  `prefix_salt` must name the model (weights + KV format).
        self.prefix_cache, self.prefix_salt = prefix_cache, prefix_salt
        self.prefix_stats = {"lookups": 0, "blocks_hit": 0, "blocks_stored": 0, "tokens_skipped": 0}
        self.session_cache = None  # a SessionSnapshotCache: per-conversation KV (+ recurrent state) snapshots
        cfg = model.cfg
        has_head = getattr(model.w, "mtp", None) is not None
        self.mtp_k = mtp_draft_tokens if has_head else 0
        self.mtp_depth = self.mtp_k  # drafts the next cycle verifies (columns 0 .. depth-1 of `draft` are primed)
        self.depth_controller = None
        if mtp_dynamic_depth and self.mtp_k > 1:
            from .mtp_policy import CycleDepthController
            self.depth_controller = CycleDepthController(self.mtp_k)
        self.device = torch.device(device) if device is not None else model.w.embed.device
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        pages_per_seq = (max_seq_len + PAGE_SIZE - 1) // PAGE_SIZE
        if num_pages is None:
            num_pages = max_batch * pages_per_seq + 1
        self.cache = PagedKVCache(layers=getattr(model, "local_layers", cfg.num_layers) + (1 if has_head else 0), kv_heads=model.hk, head_dim=cfg.head_dim, num_pages=num_pages,
                                  max_seqs=max_batch, max_pages_per_seq=pages_per_seq, device=self.device)
        dev = self.device
        self.input_ids = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.seq_lens = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.slots = torch.full((max_batch,), -1, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.active = torch.ones(max_batch, dtype=torch.int32, device=dev)
        # per-row sampling record, 32 bytes: temperature f32, top_k i32, top_p f32, presence f32, frequency f32,
        # repetition f32, seed u64 (the layout the sampling kernel reads)
        self.sample_rows = torch.zeros((max_batch, 8), dtype=torch.int32, device=dev)
        self.sample_work: torch.Tensor | None = None
        self.verify_work: torch.Tensor | None = None  # scratch of the speculative verification draw
        self.use_graphs = use_graphs and dev.type == "cuda"
        self.graphs: dict[tuple[int, bool, int], torch.cuda.CUDAGraph] = {}
        self.launches_per_step: dict[int, int] = {}
        self.row_seq: dict[int, int] = {}
        self.row_len: dict[int, int] = {}  # host mirror of seq_lens for page management
        self.row_stochastic: dict[int, bool] = {}
        self.row_constraint: dict[int, object] = {}  # row -> grammar state of a structured-output request
        self.logit_bias: torch.Tensor | None = None  # [max_batch, vocabulary] bf16, allocated by the first such request
        self._token_bytes, self._constraint_vocab, self._constraint_stop = None, None, ()
        self._next_seq_id = 0
        # models with recurrent (linear-attention) state keep it per batch row
        self.rec_state = model.make_state(max_batch) if hasattr(model, "make_state") else None
        self.row_ids = torch.arange(max_batch, dtype=torch.int32, device=dev)
        self.state_slots = torch.full((max_batch,), -1, dtype=torch.int32, device=dev)
        if self.mtp_k:
            k, w = self.mtp_k, self.mtp_k + 1
            if w * (cfg.num_heads // max(1, cfg.num_kv_heads)) > 16:
                raise ValueError("the verify window (K+1 tokens x query heads per KV head) exceeds 16 attention rows")

            def i32(*shape, fill=0):
                return torch.full(shape, fill, dtype=torch.int32, device=dev)
            self.draft = i32(max_batch, k)
            self.v_ids, self.v_pos, self.v_slots = i32(max_batch * w), i32(max_batch * w), i32(max_batch * w, fill=-1)
            self.v_lens = i32(max_batch)
            self.targets, self.head_next = i32(max_batch * w), i32(max_batch * w)
            self.out_tokens, self.n_out, self.accept_row = i32(max_batch, w, fill=-1), i32(max_batch), i32(max_batch)
            self.c_tok, self.c_ids, self.c_pos, self.c_lens = i32(max_batch), i32(max_batch), i32(max_batch), i32(max_batch)
            self.c_slots = i32(max_batch, fill=-1)
            self.mtp_counters = torch.zeros(2, dtype=torch.int64, device=dev)  # drafted, accepted
            self.mtp_graphs: dict[tuple, torch.cuda.CUDAGraph] = {}
            self.mtp_cycles = 0
            # cycles at a depth d < K work on contiguous [batch, d] / [batch, d + 1] copies (the kernels index by depth)
            self.draft_d = {d: (self.draft if d == k else i32(max_batch, d)) for d in range(1, k + 1)}
            self.out_tokens_d = {d: (self.out_tokens if d == k else i32(max_batch, d + 1, fill=-1)) for d in range(1, k + 1)}
            self.last_depth = k

    # -- token constraints -------------------------------------------------------------------------------------------
    def set_token_bytes(self, token_bytes, stop_ids=()) -> None:
        """Give the engine the vocabulary's byte strings (see the tokenizers' ``token_bytes``); needed before a request
        may ask for structured output.  The trie is built on first use."""
        self._token_bytes, self._constraint_stop = token_bytes, tuple(stop_ids)
        self._constraint_vocab = None

    def _constraint_for(self, params):
        fmt = getattr(params, "response_format", None) if params is not None else None
        bias = getattr(params, "logit_bias", None) if params is not None else None
        if bias:
            from .constraints import LogitBias
            return LogitBias(bias, self._grammar_for(fmt, params))
        return self._grammar_for(fmt, params)

    def _grammar_for(self, fmt, params):
        if not fmt or getattr(self, "_token_bytes", None) is None:
            return None
        if self._constraint_vocab is None:
            from .. import native
            table = self._token_bytes() if callable(self._token_bytes) else self._token_bytes
            self._constraint_vocab = native.JsonVocabulary(list(table))
        from .constraints import make_constraint
        stops = tuple(getattr(params, "stop_token_ids", ()) or ()) or self._constraint_stop
        return make_constraint(fmt, self._constraint_vocab, stops)

    def _bias_rows(self, logits: torch.Tensor, b: int) -> torch.Tensor:
        """The persistent ``[max_batch, vocabulary]`` bias, cut to this rank's vocabulary shard of ``logits``."""
        v = logits.shape[1]
        tp = self.model.tp
        if self.logit_bias is None or self.logit_bias.shape[1] != v * tp:
            self.logit_bias = torch.zeros((self.max_batch, v * tp), dtype=torch.bfloat16, device=self.device)
        lo = self.model.w.tp_rank * v if tp > 1 else 0
        return self.logit_bias[:b, lo : lo + v]

    def _write_bias(self, rows) -> None:
        """Refresh the bias rows of ``rows`` from their grammar states (zero for rows without one)."""
        if self.logit_bias is None:
            return
        held = self.__dict__.setdefault("_bias_held", {})  # row -> the host row its device copy came from (None: zeros)
        for r in rows:
            c = self.row_constraint.get(r)
            src = None if c is None else c.bias(self.logit_bias.shape[1])
            if r in held and held[r] is src:
                continue  # same grammar state as last step (e.g. inside a string): the device row is already right
            if src is None:
                self.logit_bias[r].zero_()
            else:
                self.logit_bias[r].copy_(src, non_blocking=True)
            held[r] = src

    # -- capacity (scheduler backend protocol) ------------------------------------------------------------------
    def free_tokens(self) -> int:
        return self.cache.allocator.free_pages * self.cache.page_size

    def tokens_needed(self, tokens: int) -> int:
        ps = self.cache.page_size
        return (tokens + ps - 1) // ps * ps

    def can_grow(self, row: int) -> bool:
        """Make sure the row has a page for its next token; False when the pool is exhausted."""
        need = self.row_len[row] + 1 + self.mtp_k  # a verify window writes K rows past the next token
        if need > self.max_seq_len:
            return False
        try:
            self.cache.assign(row, self.row_seq[row], need)
            return True
        except MemoryError:
            return False

    def release(self, row: int) -> None:
        seq = self.row_seq.pop(row, None)
        if seq is not None:
            self.cache.release(seq)
        self.row_len.pop(row, None)
        self.row_stochastic.pop(row, None)
        self.row_constraint.pop(row, None)

    # -- sampling ---------------------------------------------------------------------------------------------------
    def set_sampling(self, row: int, params) -> None:
        """Install the row's sampling record (``params``: a :class:`SamplingParams`-like object or None = greedy)."""
        rec = torch.zeros(8, dtype=torch.int32)
        stochastic = bool(params is not None and getattr(params, "temperature", 0.0) > 0.0)
        if params is not None:
            f = torch.tensor([params.temperature, 0.0, params.top_p, params.presence_penalty, params.frequency_penalty,
                              params.repetition_penalty], dtype=torch.float32).view(torch.int32)
            rec[:6] = f
            rec[1] = int(params.top_k)
            rec[6:8] = torch.tensor([int(params.seed) & (2 ** 63 - 1)], dtype=torch.int64).view(torch.int32)
        else:
            rec[5] = torch.tensor([1.0]).view(torch.int32)[0]
        self.sample_rows[row] = rec.to(self.device)
        self.row_stochastic[row] = stochastic

    def _sample(self, logits: torch.Tensor, b: int, stochastic: bool) -> None:
        if not stochastic:
            self.model.sample_greedy(logits, out=self.sampled[:b])
            return
        if self.model.tp > 1:
            logits = self.model.collective.gather_columns(logits)
        if not logits.is_cuda:
            self._sample_reference(logits, b)
            return
        v = logits.shape[1]
        if self.sample_work is None or self.sample_work.shape[1] != v:
            self.sample_work = torch.empty((self.max_batch, v), dtype=torch.float32, device=self.device)
        fn = ops.lib.lib().mfq_sample
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6
        fn.restype = C.c_int
        rc = fn(logits.data_ptr(), b, v, logits.stride(0), None, self.sample_rows.data_ptr(), self.seq_lens.data_ptr(),
                self.sample_work.data_ptr(), self.sampled.data_ptr(), ops.lib.stream_ptr())
        ops.lib.check(rc, "sample")

    def _sample_reference(self, logits: torch.Tensor, b: int) -> None:
        for r in range(b):
            rec = self.sample_rows[r].cpu()
            temp, top_p = rec[:1].view(torch.float32).item(), rec[2:3].view(torch.float32).item()
            top_k = int(rec[1])
            l = logits[r].float()
            if temp <= 0:
                self.sampled[r] = int(l.argmax())
                continue
            l = l / temp
            if 0 < top_k < l.numel():
                l = l.masked_fill(l < l.topk(top_k).values[-1], float("-inf"))
            p = torch.softmax(l, -1)
            if top_p < 1:
                sp, si = p.sort(descending=True)
                keep = (sp.cumsum(0) - sp) < top_p
                mask = torch.zeros_like(p, dtype=torch.bool).scatter_(0, si[keep], True)
                p = torch.where(mask, p, torch.zeros_like(p))
            g = torch.Generator().manual_seed(int(rec[6:8].view(torch.int64)) + int(self.seq_lens[r]))
            self.sampled[r] = int(torch.multinomial(p / p.sum(), 1, generator=g))

    # -- prefill -------------------------------------------------------------------------------------------------
    def prefill(self, row: int, token_ids, params=None, session: str | None = None, generated: int = 0) -> int:
        """Run the prompt of batch row ``row`` through the model; returns the first generated token id and leaves
        the row ready for decode (``seq_lens[row]`` = prompt length, ``sampled[row]`` = first token).  With ``session``
        and a :attr:`session_cache`, the history of that conversation is restored from its snapshot when the prompt
        extends it.  ``generated``: how many trailing tokens of ``token_ids`` the model itself produced earlier (a
        replayed request); a token constraint re-reads them before it masks the next token."""
        dev = self.device
        self._bind_state()
        ids = torch.as_tensor(token_ids, dtype=torch.int32)
        n = int(ids.numel())
        if n + 1 > self.max_seq_len:
            raise ValueError(f"prompt of {n} tokens exceeds the engine's context of {self.max_seq_len}")
        if row in self.row_seq:
            self.release(row)
        seq_id = self._next_seq_id
        self._next_seq_id += 1
        self.row_seq[row] = seq_id
        try:
            self.cache.assign(row, seq_id, n + 1)
        except MemoryError:
            self.release(row)
            raise
        self.set_sampling(row, params)
        ids = ids.to(dev, non_blocking=True)
        state_slots = None
        if self.rec_state is not None:
            self.rec_state.reset(row)
            state_slots = self.row_ids[row : row + 1]
        last = torch.tensor([n - 1], dtype=torch.int32, device=dev)
        start, keys = 0, None
        if session is not None and self.session_cache is not None and not self.mtp_k:
            start = self.session_cache.restore(self, row, session, [int(t) for t in ids.tolist()])
        if start == 0:
            start, keys = self._restore_prefix(seq_id, token_ids, n)
        logits, hidden = self._prefill_span(row, seq_id, ids, start, n, state_slots)
        self._store_prefix(seq_id, keys, start)
        self.seq_lens[row] = n
        self.row_len[row] = n
        constraint = self._constraint_for(params)
        if constraint is not None:
            for t in (ids[n - generated :].tolist() if generated else ()):
                constraint.advance(int(t))
            self.row_constraint[row] = constraint
            bias = self._bias_rows(logits, self.max_batch)[row : row + 1]
            self._write_bias([row])
            logits = logits + bias
        if self.row_stochastic[row]:
            # sample row 0 of the one-row logits with this row's record
            saved_rows, saved_len = self.sample_rows[0].clone(), self.seq_lens[0].clone()
            saved_tok = self.sampled[0].clone()
            self.sample_rows[0], self.seq_lens[0] = self.sample_rows[row], n
            self._sample(logits, 1, True)
            tok = self.sampled[0].clone()
            self.sample_rows[0], self.seq_lens[0], self.sampled[0] = saved_rows, saved_len, saved_tok
            self.seq_lens[row] = n
        else:
            tok = self.model.sample_greedy(logits)[0]
        self.sampled[row] = tok
        if self.mtp_k:
            # teacher-forced priming of the head over the prompt: position i pairs hidden[i] with token i+1
            nxt = torch.cat([ids[1:n], tok.reshape(1).to(torch.int32)])
            mstep = StepBuffers(input_ids=nxt, positions=torch.arange(n, dtype=torch.int32, device=dev),
                                slots=self.cache.slots(seq_id, 0, n).to(dev), cu_seqlens=[0, n])
            mlogits, mhid = self.model.mtp_forward(mstep, self.cache, hidden, prefill=True, logits_rows=last)
            self.draft[row, 0] = self.model.sample_greedy(mlogits)[0]
            self._mtp_chain(row, row + 1, mhid[n - 1 : n].contiguous(), masked=False)
        if constraint is not None:
            constraint.advance(int(tok))
        return int(tok)

    def save_session(self, row: int, session: str, tokens) -> None:
        """Keep row ``row``'s KV pages (and recurrent state) as the snapshot of conversation ``session``.  ``tokens``
        is the conversation so far; only the part whose KV is in the cache (``seq_lens[row]`` tokens) is covered."""
        if self.session_cache is None or self.mtp_k:
            return
        n = int(self.seq_lens[row])
        self.session_cache.save(self, row, session, [int(t) for t in tokens[:n]])

    def _bind_state(self) -> None:
        """Engines that share one model object each own a recurrent state: point the model at this engine's."""
        if self.rec_state is not None:
            self.model.state = self.rec_state

    def _prefix_usable(self) -> bool:
        # recurrent state and the MTP head's priming need every prompt position: those models always prefill in full
        return self.prefix_cache is not None and self.rec_state is None and not self.mtp_k

    def _restore_prefix(self, seq_id: int, token_ids, n: int):
        """Restore the longest cached run of leading blocks into the sequence's pages.  Returns (tokens restored, keys
        of all full blocks that may be cached: at least one token is always left to compute, for the logits)."""
        if not self._prefix_usable():
            return 0, None
        pc = self.prefix_cache
        bt = pc.block_tokens
        usable = (n - 1) // bt * bt
        if usable == 0:
            return 0, None
        keys = pc.keys(torch.as_tensor(token_ids, dtype=torch.int32)[:usable].numpy(), salt=self.prefix_salt)
        self.prefix_stats["lookups"] += 1
        pages = self.cache.allocator.owned[seq_id]
        per_block = bt // self.cache.page_size
        nbytes = self.cache.page_blob_bytes(per_block)
        hit = 0
        for i in range(pc.match(keys)):
            blob = pc.get(keys[i], nbytes)
            if blob is None or blob.nbytes != nbytes:
                break
            self.cache.import_pages(pages[i * per_block : (i + 1) * per_block], blob)
            hit += 1
        self.prefix_stats["blocks_hit"] += hit
        self.prefix_stats["tokens_skipped"] += hit * bt
        return hit * bt, keys

    def _store_prefix(self, seq_id: int, keys, start: int) -> None:
        if keys is None:
            return
        pc = self.prefix_cache
        per_block = pc.block_tokens // self.cache.page_size
        pages = self.cache.allocator.owned[seq_id]
        for i in range(start // pc.block_tokens, len(keys)):
            pc.put(keys[i], self.cache.export_pages(pages[i * per_block : (i + 1) * per_block]))
            self.prefix_stats["blocks_stored"] += 1

    def _prefill_span(self, row: int, seq_id: int, ids: torch.Tensor, start: int, end: int, state_slots):
        with scope("prefill.span", self.device):
            return self._prefill_span_body(row, seq_id, ids, start, end, state_slots)

    def _prefill_span_body(self, row: int, seq_id: int, ids: torch.Tensor, start: int, end: int, state_slots):
        """Run tokens ``[start, end)`` of the row's sequence (``ids`` holds the whole prompt, on the device) through
        the model in chunks of at most ``prefill_chunk``; tokens before ``start`` must already be in the KV pages.
        Returns (logits of the last token, hidden states of the span if an MTP head needs them)."""
        dev = self.device
        tp = self.model.tp
        want_hidden = bool(self.mtp_k)
        hidden_parts, logits = [], None
        c0 = start
        while c0 < end:
            c1 = min(end, c0 + self.prefill_chunk)
            m = c1 - c0
            chunk_ids = ids[c0:c1]
            positions = torch.arange(c0, c1, dtype=torch.int32, device=dev)
            slots = self.cache.slots(seq_id, c0, m).to(dev)
            cu = [0, m]
            single = c0 == 0 and c1 == end
            if single and tp > 1 and m >= tp * 128 and m % (tp * 128) and self.rec_state is None:
                # pad to a whole number of token tiles per rank so the row-parallel GEMMs take the reduce-scatter path;
                # the pad rows form a sequence of their own and write no KV
                pad = tp * 128 - m % (tp * 128)
                chunk_ids = torch.cat([chunk_ids, torch.zeros(pad, dtype=torch.int32, device=dev)])
                positions = torch.cat([positions, torch.arange(pad, dtype=torch.int32, device=dev)])
                slots = torch.cat([slots, torch.full((pad,), -1, dtype=torch.int32, device=dev)])
                cu = [0, m, m + pad]
            step = StepBuffers(input_ids=chunk_ids, positions=positions, slots=slots, cu_seqlens=cu, state_slots=state_slots,
                               past_len=c0, block_table=self.cache.block_table[row : row + 1] if c0 else None)
            is_last = c1 == end
            rows = torch.tensor([m - 1], dtype=torch.int32, device=dev) if is_last else torch.zeros(1, dtype=torch.int32, device=dev)
            out = self.model.forward(step, self.cache, prefill=True, logits_rows=rows, gather_logits=False, return_hidden=want_hidden)
            if want_hidden:
                out, hid = out
                hidden_parts.append(hid[:m])
            if is_last:
                logits = out
            c0 = c1
        return logits, (torch.cat(hidden_parts, 0) if want_hidden else None)

    def score(self, row: int, token_ids, start: int) -> list[float]:
        """Natural-log probabilities the model gives ``token_ids[start:]``, each conditioned on everything before it:
        one chunked prefill on the free batch row ``row`` (released again afterwards; no sampling, no prefix or session
        cache).  ``start >= 1``.  The evaluation the reference serves as probability scoring
        (``mfq/server/api/routes/models.py:342-356``)."""
        dev = self.device
        self._bind_state()
        ids = torch.as_tensor(token_ids, dtype=torch.int32)
        n = int(ids.numel())
        if not 1 <= start < n:
            raise ValueError("score() needs at least one context token and one token to score")
        if n > self.max_seq_len:
            raise ValueError(f"{n} tokens exceed the engine's context of {self.max_seq_len}")
        if row in self.row_seq:
            raise ValueError(f"batch row {row} is in use")
        seq_id = self._next_seq_id
        self._next_seq_id += 1
        self.row_seq[row] = seq_id
        out: list[float] = []
        try:
            self.cache.assign(row, seq_id, n)
            ids = ids.to(dev)
            state_slots = None
            if self.rec_state is not None:
                self.rec_state.reset(row)
                state_slots = self.row_ids[row : row + 1]
            c0 = 0
            while c0 < n - 1:
                c1 = min(n, c0 + self.prefill_chunk)
                m = c1 - c0
                step = StepBuffers(input_ids=ids[c0:c1], positions=torch.arange(c0, c1, dtype=torch.int32, device=dev),
                                   slots=self.cache.slots(seq_id, c0, m).to(dev), cu_seqlens=[0, m], state_slots=state_slots,
                                   past_len=c0, block_table=self.cache.block_table[row : row + 1] if c0 else None)
                lo, hi = max(start - 1, c0), min(n - 1, c1)          # positions whose NEXT token is scored, in this chunk
                want = torch.arange(lo - c0, hi - c0, dtype=torch.int32, device=dev) if hi > lo else torch.zeros(1, dtype=torch.int32, device=dev)
                logits = self.model.forward(step, self.cache, prefill=True, logits_rows=want)
                if hi > lo:
                    logp = torch.log_softmax(logits.float(), -1)
                    out += logp.gather(1, ids[lo + 1 : hi + 1].long()[:, None])[:, 0].tolist()
                c0 = c1
        finally:
            self.release(row)
        return out

    def grow(self, row: int, tokens: int) -> None:
        self.cache.assign(row, self.row_seq[row], min(self.max_seq_len, tokens))

    # -- decode --------------------------------------------------------------------------------------------------
    def _advance(self, sampled, input_ids, positions, seq_lens, slots, table, active) -> None:
        """Feed ``sampled`` as the next input: its position, KV slot, and ``seq_lens += 1`` (active rows only)."""
        if self.device.type == "cuda":
            ops.decode_advance(sampled, input_ids, positions, seq_lens, slots, table, self.cache.page_size, active=active)
            return
        act = active.bool() if active is not None else torch.ones_like(sampled, dtype=torch.bool)
        input_ids.copy_(torch.where(act, sampled, input_ids))
        pos = seq_lens.clone()
        positions.copy_(torch.where(act, pos, positions))
        pages = table.gather(1, (pos // self.cache.page_size).long()[:, None])[:, 0]
        slots.copy_(torch.where(act, pages * self.cache.page_size + pos % self.cache.page_size, torch.full_like(pos, -1)))
        seq_lens.copy_(torch.where(act, pos + 1, pos))

    def _decode_body(self, b: int, stochastic: bool = False, constrained: bool = False, keep_head: bool = False) -> None:
        dev = self.device
        self._advance(self.sampled[:b], self.input_ids[:b], self.positions[:b], self.seq_lens[:b], self.slots[:b],
                      self.cache.block_table[:b], self.active[:b])
        state_slots = None
        if self.rec_state is not None:
            state_slots = self.state_slots[:b]
            torch.where(self.active[:b] > 0, self.row_ids[:b], torch.full_like(self.row_ids[:b], -1), out=state_slots)
        step = StepBuffers(input_ids=self.input_ids[:b], positions=self.positions[:b], slots=self.slots[:b],
                           block_table=self.cache.block_table[:b], seq_lens=self.seq_lens[:b], state_slots=state_slots)
        if dev.type == "cuda":
            self.model.attn_splits = self._splits_now(b)
        if keep_head:
            logits, hidden = self.model.forward(step, self.cache, prefill=False, gather_logits=False, return_hidden=True)
        else:
            logits = self.model.forward(step, self.cache, prefill=False, gather_logits=False)
        if constrained:
            logits += self._bias_rows(logits, b)
        self._sample(logits, b, stochastic)
        if keep_head:
            # parked speculation: the head still reads every position (its hidden state paired with the token that
            # followed), so its KV rows stay complete and draft 1 is ready when cycles resume
            mstep = StepBuffers(input_ids=self.sampled[:b], positions=self.positions[:b], slots=self.slots[:b],
                                block_table=self.cache.block_table[:b], seq_lens=self.seq_lens[:b])
            mlogits, _ = self.model.mtp_forward(mstep, self.cache, hidden, prefill=False)
            self.model.sample_greedy(mlogits, out=self.c_tok[:b])
            self.draft[:b, 0].copy_(torch.where(self.active[:b] > 0, self.c_tok[:b], self.draft[:b, 0]))  # masked rows keep theirs

    def _splits_now(self, b: int, q_len: int = 1) -> int:
        """Attention KV splits for the current contexts (host mirror of the row lengths; a graph is kept per value)."""
        from ..ops.kernels import attn_splits_for
        longest = max(self.row_len.values(), default=self.max_seq_len)
        hk = self.model.hk
        rows = max(1, getattr(self.model, "hq", hk) // hk) * q_len
        return attn_splits_for(b, hk, min(self.max_seq_len, longest), getattr(self.model.cfg, "head_dim", 128), rows)

    def enable_expert_residency_graphs(self) -> bool:
        """Let a model whose experts live behind an HBM slot arena decode inside CUDA graphs: its layers translate expert
        ids through the device slot table without asking the host, and :meth:`decode_step` settles misses after the step
        (upload, restore ``seq_lens`` / ``sampled``, run the step again).  Returns whether this engine can do that: the
        model has such layers and no draft head (draft/verify cycles would still route on the host)."""
        res = self.model.residencies() if hasattr(self.model, "residencies") else []
        if not res or self.mtp_k or self.rec_state is not None:
            return False
        self.moe_miss_count = torch.zeros(1, dtype=torch.int32, device=self.device)
        for r in res:
            r.enable_optimistic(self.moe_miss_count)
        self.residency_stats = {"steps": 0, "replays": 0, "fallbacks": 0}
        return True

    def decode_step(self, b: int, stochastic: bool = False, constrained: bool = False, keep_head: bool = False) -> None:
        """Advance the active rows among ``[0, b)`` by one token (result in ``self.sampled[:b]``, on the device).
        ``constrained``: add the rows' token-constraint bias to the logits before sampling (a graph variant of its own)."""
        if getattr(self, "moe_miss_count", None) is None:
            self._decode_step_once(b, stochastic, constrained, keep_head)
            return
        # optimistic expert residency: the step runs with the experts that are resident; if a route met an absent one,
        # bring the step's experts in and run it again from the same sequence state (its KV rows are rewritten).  A
        # missing expert upstream changes the routing downstream, so a cold start may take a replay per layer: after a
        # few the step runs in waves instead, which also leaves its experts resident.
        res = self.model.residencies()
        snap = (self.seq_lens.clone(), self.sampled.clone())
        self.residency_stats["steps"] += 1

        def restore():
            self.seq_lens.copy_(snap[0])
            self.sampled.copy_(snap[1])  # the sampler's counter is the row length: a replay draws the same token

        for r in res:
            r.optimistic = True
        try:
            for _attempt in range(self.residency_replays + 1):
                self.moe_miss_count.zero_()
                self._decode_step_once(b, stochastic, constrained, keep_head)
                if int(self.moe_miss_count.item()) == 0:
                    return
                outcomes = [r.settle() for r in res]
                restore()
                if "fallback" in outcomes:
                    break
                self.residency_stats["replays"] += 1
        finally:
            for r in res:
                r.optimistic = False
        # in waves, outside the graphs: always right, whatever the step routes to
        self.residency_stats["fallbacks"] += 1
        self._bind_state()
        self._decode_body(b, stochastic, constrained, keep_head)

    residency_replays = 3

    def _decode_step_once(self, b: int, stochastic: bool = False, constrained: bool = False, keep_head: bool = False) -> None:
        self._bind_state()
        if not self.use_graphs:
            self._decode_body(b, stochastic, constrained, keep_head)
            return
        key = (b, stochastic, self._splits_now(b)) + ((True,) if constrained else ()) + (("head",) if keep_head else ())
        g = self.graphs.get(key)
        if g is None:
            ops.Workspace.get(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            saved = (self.seq_lens.clone(), self.sampled.clone())
            saved_draft = self.draft.clone() if keep_head else None
            saved_rec = (self.rec_state.conv.clone(), self.rec_state.state.clone()) if self.rec_state is not None else None
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode_body(b, stochastic, constrained, keep_head)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(g):
                self._decode_body(b, stochastic, constrained, keep_head)
            self.launches_per_step[b] = ops.launch_count() - before
            trace("graph", "captured", rows=b, stochastic=int(stochastic), constrained=int(constrained),
                  launches=self.launches_per_step[b], graphs=len(self.graphs) + 1)
            # warm-up and capture ran real steps: roll the sequence state back (the KV rows they wrote get rewritten)
            self.seq_lens.copy_(saved[0])
            self.sampled.copy_(saved[1])
            if saved_draft is not None:
                self.draft.copy_(saved_draft)
            if saved_rec is not None:  # the recurrent state cannot be "rewritten later" like KV rows: put it back
                self.rec_state.conv.copy_(saved_rec[0])
                self.rec_state.state.copy_(saved_rec[1])
            self.graphs[key] = g
        g.replay()

    # -- MTP draft / verify ---------------------------------------------------------------------------------------
    def _mtp_chain(self, r0: int, r1: int, hid: torch.Tensor, masked: bool = True, depth: int | None = None) -> None:
        """Drafts 2..``depth`` (default K) of rows ``[r0, r1)``: the head runs on its own previous output and draft, one
        position at a time past the confirmed sequence (those KV rows are provisional and get rewritten by the next cycle)."""
        depth = self.mtp_k if depth is None else depth
        if depth < 2:
            return
        table = self.cache.block_table[r0:r1]
        tok, ids, pos, lens, slots = (t[r0:r1] for t in (self.c_tok, self.c_ids, self.c_pos, self.c_lens, self.c_slots))
        lens.copy_(self.seq_lens[r0:r1])
        for j in range(2, depth + 1):
            tok.copy_(self.draft[r0:r1, j - 2])
            self._advance(tok, ids, pos, lens, slots, table, self.active[r0:r1] if masked else None)
            step = StepBuffers(input_ids=ids, positions=pos, slots=slots, block_table=table, seq_lens=lens)
            logits, hid = self.model.mtp_forward(step, self.cache, hid, prefill=False)
            self.model.sample_greedy(logits, out=tok)
            self.draft[r0:r1, j - 1].copy_(tok)

    def _verify_targets(self, logits: torch.Tensor, draft: torch.Tensor, b: int, w: int) -> torch.Tensor:
        """The token every window position emits under the rows' sampling parameters (speculative sampling with the
        deterministic proposal of the draft head: a draft is kept with its target probability, otherwise replaced by a
        draw from the target distribution without it, so the emitted tokens follow the target distribution exactly;
        greedy rows get the arg-max).  ``logits [b * w, V]``, ``draft [b, w - 1]``; returns ``targets [b * w]``."""
        if self.model.tp > 1:
            logits = self.model.collective.gather_columns(logits)
        out = self.targets[: b * w]
        v = logits.shape[1]
        if not logits.is_cuda:
            return self._verify_targets_reference(logits, draft, b, w, out)
        if self.verify_work is None or self.verify_work.shape[1] != v:
            self.verify_work = torch.empty((self.max_batch * (self.mtp_k + 1), v), dtype=torch.float32, device=self.device)
        fn = ops.lib.lib().mfq_sample_verify
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6
        fn.restype = C.c_int
        rc = fn(logits.data_ptr(), b, w, v, logits.stride(0), self.sample_rows.data_ptr(), self.seq_lens.data_ptr(),
                draft.data_ptr(), self.verify_work.data_ptr(), out.data_ptr(), ops.lib.stream_ptr())
        ops.lib.check(rc, "sample_verify")
        return out

    def _verify_targets_reference(self, logits, draft, b: int, w: int, out: torch.Tensor) -> torch.Tensor:
        for r in range(b):
            rec = self.sample_rows[r].cpu()
            temp, top_p = rec[:1].view(torch.float32).item(), rec[2:3].view(torch.float32).item()
            top_k = int(rec[1])
            for i in range(w):
                l = logits[r * w + i].float()
                if temp <= 0:
                    out[r * w + i] = int(l.argmax())
                    continue
                l = l / temp
                if 0 < top_k < l.numel():
                    l = l.masked_fill(l < l.topk(top_k).values[-1], float("-inf"))
                p = torch.softmax(l, -1)
                if top_p < 1:
                    sp, si = p.sort(descending=True)
                    keep = (sp.cumsum(0) - sp) < top_p
                    mask = torch.zeros_like(p, dtype=torch.bool).scatter_(0, si[keep], True)
                    p = torch.where(mask, p, torch.zeros_like(p))
                p = p / p.sum()
                g = torch.Generator().manual_seed(int(rec[6:8].view(torch.int64)) + int(self.seq_lens[r]) + i)
                if i < w - 1:
                    x = int(draft[r, i])
                    if float(torch.rand((), generator=g)) < float(p[x]):
                        out[r * w + i] = x
                        continue
                    p = p.clone()
                    p[x] = 0
                    p = p / p.sum()
                out[r * w + i] = int(torch.multinomial(p, 1, generator=g))
        return out

    def _mtp_body(self, b: int, depth: int | None = None, next_depth: int | None = None, stochastic: bool = False) -> None:
        """One cycle verifying ``depth`` drafts (default K) and leaving ``next_depth`` drafts for the following one.
        ``stochastic``: rows with a temperature verify by speculative sampling instead of arg-max comparison."""
        from ..ops import mtp as mtp_ops
        k = self.mtp_k if depth is None else depth
        next_depth = k if next_depth is None else next_depth
        w = k + 1
        draft, out_tokens = self.draft_d[k], self.out_tokens_d[k]
        if draft is not self.draft:
            draft[:b].copy_(self.draft[:b, :k])
        table = self.cache.block_table[:b]
        ids, pos, slots, lens = self.v_ids[: b * w], self.v_pos[: b * w], self.v_slots[: b * w], self.v_lens[:b]
        mtp_ops.prepare(self.sampled[:b], draft[:b], self.seq_lens[:b], table, self.active[:b], ids, pos, slots, lens,
                        self.cache.page_size)
        if self.device.type == "cuda":
            self.model.attn_splits = self._splits_now(b, w)
        state_slots = None
        if self.rec_state is not None:
            state_slots = self.state_slots[:b]
            torch.where(self.active[:b] > 0, self.row_ids[:b], torch.full_like(self.row_ids[:b], -1), out=state_slots)
        step = StepBuffers(input_ids=ids, positions=pos, slots=slots, block_table=table, seq_lens=lens, q_len=w,
                           state_slots=state_slots, verify=self.rec_state is not None)
        logits, hidden = self.model.forward(step, self.cache, prefill=False, gather_logits=False, return_hidden=True)
        if stochastic:
            targets = self._verify_targets(logits, draft, b, w)
        else:
            targets = self.model.sample_greedy(logits, out=self.targets[: b * w])
        # the head sees the TRUE successor of every window position, so whatever prefix is accepted its KV rows and
        # its prediction at the last confirmed position are exact
        mstep = StepBuffers(input_ids=targets, positions=pos, slots=slots, block_table=table, seq_lens=lens, q_len=w)
        mlogits, mhid = self.model.mtp_forward(mstep, self.cache, hidden, prefill=False)
        head_next = self.model.sample_greedy(mlogits, out=self.head_next[: b * w])
        mtp_ops.accept(targets, head_next, self.active[:b], draft[:b], self.sampled[:b], self.seq_lens[:b],
                       out_tokens[:b], self.n_out[:b], self.accept_row[:b], self.mtp_counters)
        if draft is not self.draft:
            self.draft[:b, 0].copy_(draft[:b, 0])  # the first draft of the next cycle
        if self.rec_state is not None:  # recurrent layers keep the state after the last accepted window position
            self.model.commit_verify(b, w, state_slots, self.accept_row[:b])
        if next_depth > 1:
            self._mtp_chain(0, b, mtp_ops.select_rows(mhid, self.accept_row[:b], w), depth=next_depth)

    def mtp_step(self, b: int, stochastic: bool = False) -> None:
        """One draft/verify cycle for the active rows among ``[0, b)``: confirms ``n_out[r]`` in 1..K+1 tokens per
        row (``out_tokens[r, :n_out[r]]``), all state stays on the device (one CUDA graph per batch bucket)."""
        self.mtp_cycles += 1
        self._bind_state()
        depth = self.mtp_depth
        nxt = self.depth_controller.next_depth() if self.depth_controller is not None else depth
        self.last_depth, self.mtp_depth = depth, nxt
        if not self.use_graphs:
            self._mtp_body(b, depth, nxt, stochastic)
            return
        key = (b, depth, nxt) + ((True,) if stochastic else ())
        g = self.mtp_graphs.get(key)
        if g is None:
            ops.Workspace.get(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            saved = [t.clone() for t in (self.seq_lens, self.sampled, self.draft, self.mtp_counters)]
            saved_rec = (self.rec_state.conv.clone(), self.rec_state.state.clone()) if self.rec_state is not None else None
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._mtp_body(b, depth, nxt, stochastic)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(g):
                self._mtp_body(b, depth, nxt, stochastic)
            self.launches_per_step[("mtp", b) if depth == nxt == self.mtp_k else ("mtp", b, depth, nxt)] = ops.launch_count() - before
            for dst, src in zip((self.seq_lens, self.sampled, self.draft, self.mtp_counters), saved):
                dst.copy_(src)
            if saved_rec is not None:
                self.rec_state.conv.copy_(saved_rec[0])
                self.rec_state.state.copy_(saved_rec[1])
            self.mtp_graphs[key] = g
        g.replay()

    def mtp_result(self, b: int):
        """``(out_tokens [b, depth + 1], n_out [b])`` of the cycle :meth:`mtp_step` just ran (device tensors)."""
        return self.out_tokens_d[self.last_depth][:b], self.n_out[:b]

    def mtp_stats(self) -> dict:
        """Draft acceptance so far (the reference reports the same through its ``mtp_stats`` frame)."""
        drafted, accepted = (int(v) for v in self.mtp_counters.cpu()) if self.mtp_k else (0, 0)
        return {"draft_tokens": self.mtp_k, "drafted": drafted, "accepted": accepted,
                "acceptance_rate": accepted / drafted if drafted else 0.0,
                "tokens_per_cycle": 1.0 + (accepted / drafted * self.mtp_k if drafted else 0.0), "cycles": getattr(self, "mtp_cycles", 0)}

    def decode(self, rows: list[int]) -> dict:
        """Scheduler entry: advance each of ``rows`` (other rows are masked off).  Returns ``{row: token}``, or
        ``{row: [tokens]}`` when the rows decode through MTP cycles."""
        if _PROFILE_DECODE:
            import sys
            import time
            t0 = time.perf_counter()
            out = self._decode_rows(rows)
            print(f"decode_profile rows={len(rows)} tokens={sum(len(v) if isinstance(v, list) else 1 for v in out.values())} "
                  f"wall_ms={(time.perf_counter() - t0) * 1e3:.3f}", file=sys.stderr)
            return out
        with scope("decode.step", self.device):
            return self._decode_rows(rows)

    def _check_pages(self, rows) -> None:
        """A row that decodes past its reserved pages would read and write the shared null page (block-table entry 0)
        and corrupt every other row doing the same: refuse before launching."""
        ps = self.cache.page_size
        owned = self.cache.allocator.owned
        for r in rows:
            if r not in self.row_seq:
                raise RuntimeError(f"row {r} was never prefilled")
            need = self.row_len[r] + 1 + self.mtp_k
            have = len(owned.get(self.row_seq[r], ())) * ps
            if need > have:
                raise RuntimeError(f"row {r} needs KV room for {need} tokens but holds pages for {have}: "
                                   "call can_grow() / grow() before decode()")

    def _decode_rows(self, rows: list[int]) -> dict:
        b = bucket_for(max(rows) + 1)
        b = min(b, self.max_batch)
        self._check_pages(rows)
        mask = torch.zeros(self.max_batch, dtype=torch.int32)
        mask[rows] = 1
        self.active.copy_(mask.to(self.device), non_blocking=True)
        constrained = any(r in self.row_constraint for r in rows)
        if constrained:
            self._write_bias(range(b))
        stochastic = any(self.row_stochastic.get(r, False) for r in rows)
        if self.mtp_k and not constrained:
            ctl = self.mtp_controller
            mode = ctl.mode() if ctl is not None else "mtp"
            t0 = time.perf_counter()
            if mode == "plain":  # parked: one token per row, the head kept primed
                self.decode_step(b, stochastic, False, keep_head=True)
                toks = self.sampled[:b].cpu()
                for r in rows:
                    self.row_len[r] += 1
                ctl.observe("plain", len(rows), len(rows), (time.perf_counter() - t0) * 1e3)
                return {r: [int(toks[r])] for r in rows}
            self.mtp_step(b, stochastic)
            toks, counts = (t.cpu() for t in self.mtp_result(b))
            out = {}
            for r in rows:
                n = int(counts[r])
                self.row_len[r] += n
                out[r] = [int(t) for t in toks[r, :n]]
            ms = (time.perf_counter() - t0) * 1e3
            if ctl is not None:
                ctl.observe("mtp", sum(len(v) for v in out.values()), len(rows), ms)
            if self.depth_controller is not None:  # acceptance of the typical row, cost of the whole cycle
                accepted = sorted(len(v) - 1 for v in out.values())[len(out) // 2]
                self.depth_controller.observe(self.last_depth, accepted, ms)
            return out
        self.decode_step(b, stochastic, constrained)
        toks = self.sampled[:b].cpu()
        for r in rows:
            self.row_len[r] += 1
            if r in self.row_constraint:
                self.row_constraint[r].advance(int(toks[r]))
        return {r: int(toks[r]) for r in rows}

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
    def generate(self, prompts: list[torch.Tensor], max_new_tokens: int, use_mtp: bool = False) -> GenerationResult:
        """Static-batch greedy generation (all prompts prefilled, then decoded together).  ``use_mtp`` decodes by
        draft/verify cycles (the host reads the per-row confirmed counts once per cycle)."""
        b = len(prompts)
        assert b <= self.max_batch
        cuda = self.device.type == "cuda"
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if cuda else None
        if cuda:
            ev[0].record()
        for row, p in enumerate(prompts):
            self.prefill(row, p)
            self.grow(row, int(p.numel()) + max_new_tokens + 1 + 2 * self.mtp_k)
        self.active.fill_(1)
        if cuda:
            ev[1].record()
        out = torch.empty((b, max_new_tokens), dtype=torch.int32, device=self.device)
        out[:, 0] = self.sampled[:b]
        if use_mtp and self.mtp_k:
            got = [1] * b
            host = out.cpu()
            while min(got) < max_new_tokens:
                self.mtp_step(b)
                toks, counts = (t.cpu() for t in self.mtp_result(b))
                for r in range(b):
                    n = min(int(counts[r]), max_new_tokens - got[r])
                    host[r, got[r] : got[r] + n] = toks[r, :n]
                    got[r] += n
                # rows that are done stop drafting; their state no longer matters
                self.active[:b] = torch.tensor([int(g < max_new_tokens) for g in got], dtype=torch.int32).to(self.device)
            out.copy_(host)
            self.active.fill_(1)
        else:
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

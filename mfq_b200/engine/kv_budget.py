"""KV memory budget: how many 16-token pages fit, and what that means for batch and context.

A page of the FP8 cache costs ``layers * kv_heads * (2 * head_dim + 8) * 16`` bytes (codes for K and V plus one fp32
multiplier per token, head and tensor).  Hybrid models add a fixed recurrent state per batch row.  The plan never
exceeds what was asked for; when the budget is smaller it keeps the batch and shortens the shared page pool (sequences
then compete for pages and the scheduler retracts the youngest when the pool runs dry), and it refuses a budget that
cannot hold even one full-length sequence.  Reference: ``mfq/server/runtime/kv_budget.py`` and the native KV memory
manager (``cpp_runtime/backends/cuda/runtime``: vram / ram / auto placement).
"""

from __future__ import annotations

from dataclasses import dataclass

PAGE_TOKENS = 16


@dataclass
class KvPlan:
    num_pages: int
    page_bytes: int
    state_bytes: int  # recurrent state for all rows (0 for attention-only models)
    wanted_pages: int
    budget_bytes: int

    @property
    def kv_bytes(self) -> int:
        return self.num_pages * self.page_bytes

    @property
    def oversubscribed(self) -> bool:
        return self.num_pages < self.wanted_pages

    def tokens(self) -> int:
        return self.num_pages * PAGE_TOKENS


def page_bytes(layers: int, kv_heads: int, head_dim: int) -> int:
    return layers * kv_heads * (2 * head_dim + 8) * PAGE_TOKENS


def plan(*, budget_bytes: int, layers: int, kv_heads: int, head_dim: int, max_batch: int, max_seq_len: int,
         state_bytes_per_row: int = 0) -> KvPlan:
    pb = page_bytes(layers, kv_heads, head_dim)
    per_seq = (max_seq_len + PAGE_TOKENS - 1) // PAGE_TOKENS
    wanted = max_batch * per_seq + 1
    state = state_bytes_per_row * max_batch
    room = budget_bytes - state
    fit = room // pb if room > 0 else 0
    if fit < per_seq + 1:
        need = state + (per_seq + 1) * pb
        raise MemoryError(f"KV budget of {budget_bytes / 2**30:.2f} GiB cannot hold one sequence of {max_seq_len} tokens "
                          f"(needs {need / 2**30:.2f} GiB with the recurrent state of {max_batch} rows)")
    return KvPlan(int(min(wanted, fit)), pb, state, wanted, budget_bytes)


def device_budget(device, fraction: float = 0.9, reserve_bytes: int = 2 << 30) -> int:
    """Bytes of the device's currently free memory that the KV cache may take (after the weights are resident)."""
    import torch
    free, _total = torch.cuda.mem_get_info(device)
    return max(0, int(free * fraction) - reserve_bytes)

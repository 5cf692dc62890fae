"""Layer placement: contiguous ranges of transformer layers per rank, run one after the other.

The capacity-first way to fit a model that is too large for one GPU when tensor parallelism is not wanted: rank ``r``
holds the weights AND the KV pages of layers ``[l0_r, l1_r)`` only.  A step walks the stages in order; the stage owner
runs its layers on the residual stream and hands the result on (``collective.broadcast_rows(h, src=stage)``: every
rank receives it, so the embedding, the output norm, the LM head and sampling are replicated and all ranks stay
bit-identical).  There is no micro-batching and no pipeline schedule: at any moment one rank computes, exactly like
the reference's ``--layer-parallel / --layer-split`` placement (``cpp_runtime/backends/cuda/ops/cuda_execution.cpp:
823-840``, ``storage/load_options.cpp:296-325``), which is likewise mutually exclusive with tensor / expert parallelism.
The hand-off is ``rows x hidden`` bf16 per stage -- 8 KB per decoded token at hidden 4096 -- so it rides on the
collective library (NCCL broadcast on GPUs) rather than on a fused kernel.

``plan_layers`` gives the ranges: equal shares by default, or proportional to ``split`` weights (``--layer-split 3,1``
puts three quarters of the layers on rank 0, e.g. when rank 1 also holds a large LM head).
"""

from __future__ import annotations


def plan_layers(num_layers: int, ranks: int, split=None) -> list[tuple[int, int]]:
    from .. import native
    if ranks < 1 or num_layers < ranks:
        raise ValueError(f"cannot place {num_layers} layers on {ranks} ranks")
    weights = [float(x) for x in split] if split else None
    if weights is not None and (len(weights) != ranks or min(weights) <= 0):
        raise ValueError(f"--layer-split needs {ranks} positive weights")
    ranges = native.tp_plan(num_layers, ranks, weights, 1)
    if any(b <= a for a, b in ranges):
        raise ValueError(f"layer split {split} leaves a rank without layers")
    return [(int(a), int(b)) for a, b in ranges]

"""``mfq serve --tensor-parallel N``: one process per GPU, the HTTP server on rank 0.

The first invocation (no ``RANK`` in the environment) re-launches the same command line under
``python -m torch.distributed.run`` with N local ranks on 127.0.0.1.  Every rank then joins the process group, builds
its collective (fused peer-memory kernels on GPUs, ``gloo`` on CPU), loads ITS shard of the checkpoint and meets the
others; rank 0 serves HTTP with its engine behind a :class:`~mfq_b200.parallel.spmd.LeaderBackend`, the other ranks
mirror its engine calls (:func:`~mfq_b200.parallel.spmd.follower_loop`) until rank 0 shuts down.

Reference: ``mfq-runtime --tensor-parallel DEVICES --expert-parallel`` (``cpp_runtime/backends/cuda/commands/
runtime.cpp:23-58``) runs the ranks inside one process; here the launcher and the command log take that place.
"""

from __future__ import annotations

import os
import socket
import sys


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launcher_argv(argv: list[str], ranks: int, port: int | None = None) -> list[str]:
    """Command line that runs ``mfq <argv>`` once per rank."""
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
            "--master-addr", "127.0.0.1", "--master-port", str(port or free_port()), "-m", "mfq_b200.cli", *argv]


def under_launcher() -> bool:
    return "RANK" in os.environ and "WORLD_SIZE" in os.environ


class RankContext:
    """What a rank needs to load and run its shard."""

    def __init__(self, device: str) -> None:
        import torch
        import torch.distributed as dist
        from ..parallel.spmd import CommandLog
        self.rank, self.world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        local = int(os.environ.get("LOCAL_RANK", self.rank))
        cuda = device.startswith("cuda")
        if cuda:
            torch.cuda.set_device(local)
            self.device = f"cuda:{local}"
        else:
            self.device = "cpu"
        if not dist.is_initialized():
            dist.init_process_group("nccl" if cuda else "gloo")
        if cuda:
            from ..parallel.tensor_parallel import TensorParallel
            self.collective = TensorParallel(dist.group.WORLD, torch.device(self.device))
        else:
            from ..parallel.local_collective import ProcessGroupCollective
            self.collective = ProcessGroupCollective()
        # the command log gets a store of its own (one port above the rendezvous), so it outlives collective timeouts
        port = int(os.environ.get("MFQ_SPMD_PORT") or int(os.environ["MASTER_PORT"]) + 1)
        store = dist.TCPStore("127.0.0.1", port, self.world, is_master=self.rank == 0, wait_for_workers=True)
        self.log = CommandLog(store, self.rank, self.world)

    def finish(self) -> None:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()

"""Peer-mapped device buffers: every rank allocates one, all ranks map all of them (CUDA IPC over NVLink).

The fused compute+collective kernels receive the resulting pointer tables and load/store peer memory directly.
Buffers start zeroed.  Creation is collective: every rank of the group must call it in the same order.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops.lib import lib


class _RawCudaMemory:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can alias it without copying."""

    def __init__(self, address: int, nbytes: int, owner) -> None:
        self.owner = owner  # keeps the allocation alive as long as the tensor
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3,
                                         "strides": None}


def alias_device_memory(address: int, nbytes: int, device: torch.device, owner=None) -> torch.Tensor:
    """uint8 tensor over ``[address, address + nbytes)`` of ``device`` (zero-copy)."""
    with torch.cuda.device(device):
        return torch.as_tensor(_RawCudaMemory(address, nbytes, owner), device=device)


class PeerBuffer:
    def __init__(self, group, nbytes: int, device: torch.device) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = nbytes
        self.device = device
        L = lib()
        L.mfq_ipc_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]
        L.mfq_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        L.mfq_ipc_close.argtypes = [C.c_void_p]
        L.mfq_ipc_free.argtypes = [C.c_void_p]
        with torch.cuda.device(device):
            own = C.c_void_p()
            handle = C.create_string_buffer(64)
            rc = L.mfq_ipc_alloc(nbytes, C.byref(own), handle)
            if rc != 0:
                raise RuntimeError(f"peer buffer allocation failed ({rc})")
            handles: list = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.ptrs: list[int] = []
            self._opened: list[int] = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(own.value)
                    continue
                p = C.c_void_p()
                if L.mfq_ipc_open(h, C.byref(p)) != 0:
                    raise RuntimeError(f"rank {self.rank}: cannot map the buffer of rank {r} (no peer access?)")
                self.ptrs.append(p.value)
                self._opened.append(p.value)
        self._own = own.value
        dist.barrier(group=group)

    def local_tensor(self) -> torch.Tensor:
        """This rank's own allocation as a uint8 tensor (zero-copy alias; peers write into it)."""
        return alias_device_memory(self._own, self.nbytes, self.device, owner=self)

    def table(self):
        """ctypes array of ``world`` device pointers (index = rank)."""
        return (C.c_void_p * self.world)(*self.ptrs)

    def offset_table(self, byte_offset: int):
        return (C.c_void_p * self.world)(*[p + byte_offset for p in self.ptrs])

    def close(self) -> None:
        L = lib()
        for p in self._opened:
            L.mfq_ipc_close(p)
        self._opened = []
        if self._own:
            L.mfq_ipc_free(self._own)
            self._own = 0

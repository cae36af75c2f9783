"""Symmetric heap over NVLink peer memory.

Every rank of a model-parallel group allocates one buffer of the same size with PyTorch's
symmetric-memory allocator and exchanges handles once (rendezvous); afterwards each rank holds
a device pointer to every peer's buffer.  All kernel-issued communication (all-gather by peer
stores, reduce-scatter epilogues, vocab-parallel exchanges, cross-GPU particle copies) addresses
peers as ``peer_base[rank] + offset`` with the same offset on every rank, and synchronises through
monotonically increasing 64-bit counters that live in the heap as well.  The heap exists before any
CUDA graph is captured, so captured kernels can carry the peer addresses as plain arguments.
"""
from __future__ import annotations

import os
from typing import Dict, List, Tuple

import torch


class SymmHeap:
    def __init__(self, nbytes: int, device: torch.device, group, rank: int, world: int):
        # No kernel here uses multimem / NVLS, and a rank that exits while its buffer is bound to an NVLink multicast
        # object can fault its peers, so PyTorch's rendezvous is told not to create that binding.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.nbytes = int(nbytes)
        self.device = device
        self.rank, self.world = rank, world
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        assert self.ptrs[rank] == self.local.data_ptr()
        self._cursor = 0
        self._named: Dict[str, Tuple[int, int]] = {}
        torch.cuda.synchronize(device)
        self.handle.barrier()

    def alloc(self, name: str, nbytes: int, align: int = 256) -> int:
        """Reserve ``nbytes`` at the same offset on every rank (all ranks must allocate in the same order)."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted allocating {name} ({nbytes} bytes)")
        self._cursor = off + nbytes
        self._named[name] = (off, nbytes)
        return off

    def view(self, off: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[off:off + nbytes].view(dtype).view(*shape)

    def local_ptr(self, off: int) -> int:
        return self.ptrs[self.rank] + off

    def barrier(self) -> None:
        torch.cuda.synchronize(self.device)
        self.handle.barrier()


class FakeHeap:
    """Single-process stand-in: ``world`` ranks share one CUDA device, each with its own buffer.
    Lets the peer-store kernels run as one stream-ordered sequence of launches (never as concurrent
    spinning kernels) for single-GPU tests of the multi-rank data paths."""

    def __init__(self, nbytes: int, device, world: int):
        self.nbytes, self.world, self.device = int(nbytes), world, torch.device(device)
        self.buffers = [torch.zeros(self.nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        self.ptrs = [b.data_ptr() for b in self.buffers]
        self._cursor = 0

    def alloc(self, name: str, nbytes: int, align: int = 256) -> int:
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(name)
        self._cursor = off + nbytes
        return off

    def view(self, rank: int, off: int, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buffers[rank][off:off + nbytes].view(dtype).view(*shape)

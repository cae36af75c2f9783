"""Distributed bootstrap: one process per GPU, ``torch.distributed`` for the plumbing.

NCCL carries bulk / rare collectives and is the baseline the fused kernels are measured
against; a gloo group carries host-side object broadcasts (request fan-out to the ranks
of one model-parallel group) and is the backend of every CPU multi-process test.
Rendezvous is always on 127.0.0.1.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.distributed as dist


@dataclass
class Comm:
    rank: int
    world: int
    group_size: int                 # ranks cooperating on one request stream (tp * particle-parallel)
    group_rank: int
    replica: int
    device_group: Any = None        # NCCL (or gloo on CPU) group of this model-parallel group
    host_group: Any = None          # gloo group of the same ranks
    backend: str = "gloo"
    symm: Any = None                # symmetric-memory heap (CUDA only)

    @classmethod
    def init(cls, rank: int, world: int, args, port: int, group_size: Optional[int] = None,
             timeout_s: float = 600.0) -> "Comm":
        group_size = group_size or world
        use_cuda = args.device != "cpu" and torch.cuda.is_available()
        backend = "nccl" if use_cuda else "gloo"
        # symmetric-memory heaps are used with plain peer loads/stores only: keep them off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", str(port))
            kw = {}
            if use_cuda:
                kw["device_id"] = torch.device("cuda", args.base_gpu_id + rank)
            dist.init_process_group(backend=backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                    world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kw)
        replica, group_rank = divmod(rank, group_size)
        dev_group = host_group = None
        for r in range(world // group_size):
            ranks = list(range(r * group_size, (r + 1) * group_size))
            g = dist.new_group(ranks, backend=backend)
            h = dist.new_group(ranks, backend="gloo")
            if r == replica:
                dev_group, host_group = g, h
        return cls(rank, world, group_size, group_rank, replica, dev_group, host_group, backend)

    @classmethod
    def from_env(cls, args=None, group_size: Optional[int] = None) -> "Comm":
        """For ``torchrun`` launches: RANK / WORLD_SIZE / MASTER_PORT come from the environment."""
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        port = int(os.environ.get("MASTER_PORT", "29500"))

        class _A:
            device = "auto"
            base_gpu_id = 0
        return cls.init(rank, world, args or _A(), port, group_size)

    def broadcast_objects(self, objs: List[Any], src_group_rank: int = 0) -> List[Any]:
        box = [objs if self.group_rank == src_group_rank else None]
        src = self.replica * self.group_size + src_group_rank
        dist.broadcast_object_list(box, src=src, group=self.host_group)
        return box[0]

    def barrier(self) -> None:
        dist.barrier(group=self.host_group)

    def shutdown(self) -> None:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass

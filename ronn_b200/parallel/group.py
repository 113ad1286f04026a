"""Process-group bootstrap and the library-collective communicator.

One process per GPU (torchrun); NCCL over NVLink/NVSwitch on GPUs, gloo on CPU for the host-side
tests.  ``TPComm`` is the baseline communicator of the tensor-parallel decoder: plain library
all-reduce / all-gather.  The reference has no communication backend at all (its "multi-GPU" layer
picks one device per sub-graph and simulates transfers with sleeps:
crates/ronn-providers/src/gpu/provider.rs:226-249, gpu/memory_manager.rs:411-413).
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


def init_distributed(backend: Optional[str] = None, timeout_s: int = 600):
    """Initialise torch.distributed from the torchrun environment.  Returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1:
        return 0, 1, 0
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


class TPComm:
    """Library collectives over a process group."""
    fused = False

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.calls = 0

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(x, group=self.group)
            self.calls += 1
        return x

    def all_gather_small(self, x: torch.Tensor) -> torch.Tensor:
        """[...] -> [world, ...]"""
        if self.world == 1:
            return x.unsqueeze(0)
        flat = x.contiguous().reshape(-1)
        out = torch.empty(self.world * flat.numel(), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, flat, group=self.group)
        self.calls += 1
        return out.reshape((self.world,) + tuple(x.shape))

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        """[m, n] shards -> [world*m, n]"""
        if self.world == 1:
            return x
        out = torch.empty((self.world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        """[world*m, n] partial sums -> this rank's [m, n] of the total"""
        if self.world == 1:
            return x
        per = x.shape[0] // self.world
        if dist.get_backend(self.group) == "gloo":          # no reduce-scatter there: sum everything, keep the shard
            full = x.contiguous().clone()
            dist.all_reduce(full, group=self.group)
            return full[self.rank * per:(self.rank + 1) * per].contiguous()
        out = torch.empty((per,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else "cpu"
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

"""Multi-GPU memory manager with real peer transfers
(crates/ronn-providers/src/gpu/memory_manager.rs:16-737: per-device pools, P2P connectivity matrix,
``transfer_between_devices``, sync strategies and an event log, ``optimize_memory_layout``; the
reference only keeps accounts and simulates transfers with sleeps).  Buffers are torch CUDA tensors
from the caching allocator; a transfer is a peer copy over NVLink when peer access exists, else a
staged copy through pinned host memory."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..api.errors import ProviderError


class SyncStrategy(enum.Enum):
    EXPLICIT = "explicit"
    AUTOMATIC = "automatic"
    STREAM_BASED = "stream_based"


@dataclass
class SyncEvent:
    kind: str
    src: int
    dst: int
    nbytes: int
    seconds: float
    path: str


@dataclass
class MemoryPoolStats:
    allocated_bytes: int = 0
    peak_bytes: int = 0
    allocation_count: int = 0


@dataclass
class MultiGpuMemoryConfig:
    enable_p2p: bool = True
    sync_strategy: SyncStrategy = SyncStrategy.AUTOMATIC
    per_device_limit: Optional[int] = None


class P2PConnectivityMatrix:
    def __init__(self, n: int, matrix: Optional[List[List[bool]]] = None):
        self.n = n
        if matrix is None:
            matrix = [[False] * n for _ in range(n)]
            if torch.cuda.is_available():
                for a in range(n):
                    for b in range(n):
                        if a != b:
                            try:
                                matrix[a][b] = torch.cuda.can_device_access_peer(a, b)
                            except Exception:
                                matrix[a][b] = False
        self.matrix = matrix

    def can_access(self, a: int, b: int) -> bool:
        return a == b or self.matrix[a][b]


class MultiGpuMemoryManager:
    def __init__(self, device_ids: List[int], config: MultiGpuMemoryConfig = None,
                 connectivity: Optional[P2PConnectivityMatrix] = None):
        self.device_ids = list(device_ids)
        self.config = config or MultiGpuMemoryConfig()
        self.connectivity = connectivity or P2PConnectivityMatrix(max(device_ids) + 1 if device_ids else 0)
        self.pools: Dict[int, MemoryPoolStats] = {d: MemoryPoolStats() for d in device_ids}
        self.events: List[SyncEvent] = []

    def allocate(self, device: int, shape, dtype=torch.float32) -> torch.Tensor:
        if device not in self.pools:
            raise ProviderError(f"device {device} is not managed")
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes == 0:
            raise ProviderError("Cannot allocate zero-sized tensor")
        p = self.pools[device]
        if self.config.per_device_limit is not None and p.allocated_bytes + nbytes > self.config.per_device_limit:
            raise ProviderError(f"device {device} memory limit exceeded")
        dev = torch.device("cuda", device) if torch.cuda.is_available() else torch.device("cpu")
        t = torch.empty(tuple(shape), dtype=dtype, device=dev)
        p.allocated_bytes += nbytes
        p.peak_bytes = max(p.peak_bytes, p.allocated_bytes)
        p.allocation_count += 1
        return t

    def release(self, device: int, t: torch.Tensor) -> None:
        p = self.pools[device]
        p.allocated_bytes = max(p.allocated_bytes - t.numel() * t.element_size(), 0)

    def transfer_between_devices(self, t: torch.Tensor, src: int, dst: int) -> torch.Tensor:
        t0 = time.perf_counter()
        if not torch.cuda.is_available():
            out, path = t.clone(), "host"
        elif src == dst:
            out, path = t, "local"
        elif self.config.enable_p2p and self.connectivity.can_access(dst, src):
            out = torch.empty_like(t, device=torch.device("cuda", dst))
            out.copy_(t, non_blocking=self.config.sync_strategy != SyncStrategy.EXPLICIT)
            path = "p2p"
        else:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            host.copy_(t)
            out = host.to(torch.device("cuda", dst))
            path = "host_staged"
        if torch.cuda.is_available() and self.config.sync_strategy == SyncStrategy.AUTOMATIC and path not in ("local",):
            torch.cuda.synchronize(dst)
        self.events.append(SyncEvent("transfer", src, dst, t.numel() * t.element_size(), time.perf_counter() - t0, path))
        return out

    def optimize_memory_layout(self) -> int:
        """Device with the most free managed memory (target for the next large allocation)."""
        return min(self.device_ids, key=lambda d: self.pools[d].allocated_bytes)

    def global_stats(self) -> Dict[str, int]:
        return {"allocated_bytes": sum(p.allocated_bytes for p in self.pools.values()),
                "peak_bytes": sum(p.peak_bytes for p in self.pools.values()),
                "allocations": sum(p.allocation_count for p in self.pools.values()), "transfers": len(self.events)}

"""Device memory pool of the GPU provider: size-keyed reuse of freed blocks, a byte limit, statistics.

The reference's GPU allocator keeps freed allocations in a pool keyed by size, hands a pooled block to a request when
the block is at most twice the requested size, caps the pool at 256 MB and hands out ids that it resolves through a
registry (crates/ronn-providers/src/gpu/allocator.rs:16-64,144-225,265-370).  Here a block is a ``torch.uint8``
tensor on the pool's device (so the bytes come from the process's caching allocator and are visible to every kernel
and library call), the id is its device address, and ``GpuProviderConfig.memory_limit`` bounds live plus pooled
bytes: a request that would cross it first drops pooled blocks and only then fails.  The pool holds what the provider
itself keeps alive across runs (the static input buffers of CUDA-graph sessions, workspaces a caller asks for);
transient activations of a run come from the caching allocator directly.  Works on any torch device, which is how the
CPU test suite exercises it.
"""
from __future__ import annotations

import bisect
import threading
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..api.errors import ProviderError
from ..core.types import DataType, MemoryInfo, MemoryType, TensorBuffer
from .allocator import PoolStats
from .base import TensorAllocator


class DevicePool(TensorAllocator):
    def __init__(self, device, limit_bytes: Optional[int] = None, max_pool_bytes: int = 256 << 20,
                 reuse_factor: float = 2.0, granularity: int = 512):
        if granularity <= 0 or granularity & (granularity - 1):
            raise ProviderError("pool granularity must be a power of two")
        if reuse_factor < 1.0:
            raise ProviderError("reuse factor must be at least 1")
        self.device = torch.device(device)
        self.limit_bytes = limit_bytes
        self.max_pool_bytes = int(max_pool_bytes)
        self.reuse_factor = float(reuse_factor)
        self.granularity = int(granularity)
        self._lock = threading.Lock()
        self._live: Dict[int, torch.Tensor] = {}                 # address -> block handed out
        self._free_sizes: List[int] = []                         # sorted sizes of the pooled blocks
        self._free: List[torch.Tensor] = []                      # pooled blocks, same order
        self._live_bytes = self._pooled_bytes = self._peak = 0
        self._hits = self._misses = self._allocs = self._frees = 0

    # ------------------------------------------------------------------ blocks
    def _round(self, nbytes: int) -> int:
        g = self.granularity
        return (int(nbytes) + g - 1) // g * g

    def _take(self, need: int) -> torch.Tensor:
        """A block of at least `need` bytes: the smallest pooled one within the reuse factor, else a new one."""
        i = bisect.bisect_left(self._free_sizes, need)
        if i < len(self._free_sizes) and self._free_sizes[i] <= need * self.reuse_factor:
            self._hits += 1
            size = self._free_sizes.pop(i)
            self._pooled_bytes -= size
            return self._free.pop(i)
        self._misses += 1
        if self.limit_bytes is not None:
            over = self._live_bytes + self._pooled_bytes + need - self.limit_bytes
            while over > 0 and self._free:                       # largest pooled blocks go first
                size = self._free_sizes.pop()
                self._free.pop()
                self._pooled_bytes -= size
                over -= size
            if over > 0:
                raise ProviderError(f"device pool limit of {self.limit_bytes} bytes reached: {self._live_bytes} live, "
                                    f"{need} requested")
        try:
            return torch.empty(need, dtype=torch.uint8, device=self.device)
        except RuntimeError as e:                                # out of device memory: give the pool back and retry once
            if not self._free:
                raise ProviderError(f"device allocation of {need} bytes failed: {e}") from e
            self._free.clear()
            self._free_sizes.clear()
            self._pooled_bytes = 0
            return torch.empty(need, dtype=torch.uint8, device=self.device)

    def acquire(self, nbytes: int) -> torch.Tensor:
        """A ``uint8`` block of at least `nbytes` (rounded up to the granularity); give it back with ``release``."""
        if nbytes <= 0:
            raise ProviderError("cannot allocate a zero-size buffer")
        need = self._round(nbytes)
        with self._lock:
            blk = self._take(need)
            self._live[blk.data_ptr()] = blk
            self._live_bytes += blk.numel()
            self._allocs += 1
            self._peak = max(self._peak, self._live_bytes + self._pooled_bytes)
        return blk

    def release(self, block) -> None:
        """Return a block (the tensor, any view that starts at its address, or the address)."""
        if not isinstance(block, int) and block.numel() == 0:
            return                                               # empty tensors never took a block
        addr = block if isinstance(block, int) else block.data_ptr()
        with self._lock:
            blk = self._live.pop(addr, None)
            if blk is None:
                raise ProviderError(f"buffer 0x{addr:x} does not belong to this pool (or was released twice)")
            size = blk.numel()
            self._live_bytes -= size
            self._frees += 1
            if self._pooled_bytes + size <= self.max_pool_bytes:
                i = bisect.bisect_left(self._free_sizes, size)
                self._free_sizes.insert(i, size)
                self._free.insert(i, blk)
                self._pooled_bytes += size

    def tensor(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A tensor of `shape` / `dtype` backed by a pool block (release it with ``release(tensor)``)."""
        n = 1
        for s in shape:
            n *= int(s)
        if n == 0:
            return torch.empty(list(shape), dtype=dtype, device=self.device)
        item = torch.empty((), dtype=dtype).element_size()
        blk = self.acquire(n * item)
        return blk[: n * item].view(dtype).reshape(list(shape))

    # ------------------------------------------------------------------ TensorAllocator
    def allocate(self, shape: Sequence[int], dtype: DataType) -> TensorBuffer:
        n = 1
        for s in shape:
            n *= int(s)
        blk = self.acquire(n * dtype.itemsize)
        mt = MemoryType.DEVICE if self.device.type == "cuda" else MemoryType.SYSTEM
        return TensorBuffer(blk.data_ptr(), blk.numel(), 256 if self.device.type == "cuda" else 64, mt)

    def deallocate(self, buf: TensorBuffer) -> None:
        self.release(int(buf.ptr))

    def get_memory_info(self) -> MemoryInfo:
        if self.limit_bytes is not None:
            total = self.limit_bytes
        elif self.device.type == "cuda":
            total = torch.cuda.get_device_properties(self.device).total_memory
        else:
            total = 0
        with self._lock:
            return MemoryInfo(total, self._live_bytes + self._pooled_bytes, self._peak)

    # ------------------------------------------------------------------ statistics
    def stats(self) -> PoolStats:
        with self._lock:
            return PoolStats(self._hits, self._misses, self._live_bytes, self._peak, self._pooled_bytes,
                             len(self._free), self._allocs, self._frees, len(self._live))

    def clear_pools(self) -> Tuple[int, int]:
        """Drop every pooled block; returns (blocks, bytes) given back to the caching allocator."""
        with self._lock:
            n, b = len(self._free), self._pooled_bytes
            self._free.clear()
            self._free_sizes.clear()
            self._pooled_bytes = 0
        return n, b

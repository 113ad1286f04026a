"""Host allocators over the native pool (crates/ronn-providers/src/allocator.rs:45-505,
crates/ronn-providers/src/cpu/allocator.rs:16-220, crates/ronn-core/src/memory_pool.rs:74-257,
crates/ronn-providers/src/bitnet/allocator.rs:16-205)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from .. import _native
from ..api.errors import ProviderError
from ..core.types import DataType, MemoryInfo, MemoryType, TensorBuffer
from .base import TensorAllocator


def calculate_tensor_size(shape: Sequence[int], dtype: DataType) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * dtype.itemsize


def get_alignment_requirement(dtype: DataType) -> int:
    return max(dtype.itemsize, 1)


def get_simd_alignment() -> int:
    lvl = _native.host().ronn_cpu_simd_level()
    return 64 if lvl >= 2 else (32 if lvl >= 1 else 16)


@dataclass
class PoolStats:
    hits: int
    misses: int
    allocated_bytes: int
    peak_bytes: int
    pooled_bytes: int
    pooled_buffers: int
    allocation_count: int
    deallocation_count: int
    live_buffers: int

    @property
    def hit_rate(self) -> float:
        t = self.hits + self.misses
        return self.hits / t if t else 0.0


class _NativePool(TensorAllocator):
    memory_type = MemoryType.SYSTEM

    def __init__(self, granularity: int, alignment: int, max_per_bucket: int, max_pool_bytes: int,
                 max_total_buffers: int = 0):
        self._lib = _native.host()
        self._h = self._lib.ronn_pool_new(granularity, alignment, max_per_bucket, max_pool_bytes, max_total_buffers)
        if not self._h:
            raise ProviderError(f"invalid allocator configuration (alignment {alignment})")
        self.alignment = alignment

    def allocate_bytes(self, nbytes: int) -> TensorBuffer:
        if nbytes <= 0:
            raise ProviderError("Cannot allocate zero-sized tensor")
        p = self._lib.ronn_pool_alloc(self._h, int(nbytes))
        if not p:
            raise ProviderError(f"allocation of {nbytes} bytes failed")
        return TensorBuffer(int(p), int(nbytes), self.alignment, self.memory_type)

    def allocate(self, shape, dtype: DataType = DataType.F32) -> TensorBuffer:
        return self.allocate_bytes(calculate_tensor_size(shape, dtype))

    def deallocate(self, buf: TensorBuffer) -> None:
        if self._lib.ronn_pool_release(self._h, C.c_void_p(buf.ptr)) != 0:
            raise ProviderError("deallocate: unknown buffer (double free?)")

    def as_numpy(self, buf: TensorBuffer, dtype=np.uint8):
        n = buf.size // np.dtype(dtype).itemsize
        return np.ctypeslib.as_array(C.cast(C.c_void_p(buf.ptr), C.POINTER(C.c_uint8)), (buf.size,)).view(dtype)[:n]

    def stats(self) -> PoolStats:
        out = (C.c_uint64 * 9)()
        self._lib.ronn_pool_stats(self._h, out)
        return PoolStats(*[int(x) for x in out])

    def get_memory_info(self) -> MemoryInfo:
        s = self.stats()
        return MemoryInfo(total_bytes=2 ** 63 - 1, allocated_bytes=s.allocated_bytes, peak_bytes=s.peak_bytes)

    def clear_pools(self) -> None:
        self._lib.ronn_pool_clear(self._h)

    def bucket_size(self, nbytes: int) -> int:
        return int(self._lib.ronn_pool_bucket_size(self._h, nbytes))

    def __del__(self):
        try:
            if self._h:
                self._lib.ronn_pool_free(self._h)
                self._h = None
        except Exception:
            pass


class SystemMemoryAllocator(_NativePool):
    """No pooling: every release goes back to the system."""
    def __init__(self):
        super().__init__(1, 16, 0, 0)


class AlignedMemoryAllocator(_NativePool):
    def __init__(self, alignment: int = 64):
        super().__init__(1, alignment, 0, 0)


@dataclass
class PoolConfig:
    max_buffers_per_bucket: int = 64
    max_pool_size: int = 256 * 1024 * 1024
    bucket_granularity: int = 64


class PooledMemoryAllocator(_NativePool):
    def __init__(self, config: PoolConfig = None):
        self.config = config or PoolConfig()
        super().__init__(self.config.bucket_granularity, 64, self.config.max_buffers_per_bucket,
                         self.config.max_pool_size)

    def hit_rate(self) -> float:
        return self.stats().hit_rate


class MemoryPool(_NativePool):
    """Power-of-two size classes, 16 buffers per class, 256 buffers overall."""
    def __init__(self, max_per_class: int = 16, max_total: int = 256):
        super().__init__(0, 64, max_per_class, 1 << 40, max_total)


_GLOBAL_POOL = None


def global_pool() -> MemoryPool:
    global _GLOBAL_POOL
    if _GLOBAL_POOL is None:
        _GLOBAL_POOL = MemoryPool()
    return _GLOBAL_POOL


class BitNetAllocator(_NativePool):
    """Packed-size accounting: BOOL tensors take 1 bit per element, U8 (ternary codes) 2 bits; 32-byte aligned."""
    def __init__(self):
        super().__init__(32, 32, 32, 64 * 1024 * 1024)

    @staticmethod
    def packed_size(shape, dtype: DataType) -> int:
        n = 1
        for s in shape:
            n *= int(s)
        if dtype == DataType.BOOL:
            return (n + 7) // 8
        if dtype == DataType.U8:
            return (n + 3) // 4
        return n * dtype.itemsize

    def allocate(self, shape, dtype: DataType = DataType.U8) -> TensorBuffer:
        return self.allocate_bytes(self.packed_size(shape, dtype))

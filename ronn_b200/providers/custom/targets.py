"""Providers for targets other than the B200: NPU- and TPU-style accelerators and the WebAssembly target.

The reference ships example NPU / TPU providers whose compile and execute steps are simulated with sleeps
(crates/ronn-providers/src/custom/example_npu.rs:23-389, example_tpu.rs:23-646) and a browser provider
(crates/ronn-providers/src/wasm/provider.rs:23-330, kernels.rs:14-190, allocator.rs:15-247, bridge.rs:172-305).
Here the NPU and TPU providers are built on the plugin contracts (``interface.py``) over a host-emulated device
(``host_device.py``): they keep the reference's configuration surface, compute real results with the part's numeric
personality (int8 weights for the NPU, bfloat16 compute for the TPU) and account memory in a bounded device arena.
The WebAssembly provider keeps what is host code in the reference and makes it real: the linear-memory page allocator
with its limit, the LRU model cache with expiry, and scalar / 128-bit-SIMD-shaped kernels on the CPU operator
registry restricted to the target's operator list; the JavaScript bridge has no counterpart outside a browser.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List

import torch

from ...api.errors import ProviderError
from ...core.types import (DataType, MemoryType, PerformanceProfile, ProviderCapability, ProviderType)
from ..base import ExecutionProvider, build_kernel
from .host_device import HostEmulatedProvider, npu_capability, tpu_capability
from .interface import CompilationOptions, CustomProviderAdapter


@dataclass
class WasmProviderConfig:
    memory_limit_bytes: int = 256 * 1024 * 1024
    enable_simd: bool = True
    enable_kernel_caching: bool = True
    enable_web_workers: bool = False
    worker_count: int = 4
    optimization_level: int = 2
    enable_model_caching: bool = True
    cache_expiry_hours: int = 24
    max_cache_size: int = 128 * 1024 * 1024


class PowerMode(enum.Enum):
    PERFORMANCE = "performance"
    BALANCED = "balanced"
    POWER_SAVER = "power_saver"


@dataclass
class NpuConfig:
    device_id: str = "npu0"
    memory_pool_size: int = 2 * 1024 ** 3
    enable_quantization: bool = True
    target_precision: str = "int8"
    power_mode: PowerMode = PowerMode.BALANCED
    compiler_flags: List[str] = field(default_factory=list)
    enable_profiling: bool = False


@dataclass
class TpuConfig:
    core_count: int = 8
    generation: str = "V4"
    memory_per_core: int = 32 * 1024 ** 3
    enable_bfloat16: bool = True
    matrix_unit_size: int = 128
    interconnect: str = "ICI"
    xla_config: Dict[str, str] = field(default_factory=dict)
    pod_config: Dict[str, str] = field(default_factory=dict)



class NpuProvider(CustomProviderAdapter):
    """NPU-style part: int8 symmetric weights, fp32 activations, a bounded device arena."""
    name = "NpuProvider"

    def __init__(self, config: NpuConfig = None):
        self.config = config or NpuConfig()
        hw = HostEmulatedProvider("NpuProvider", npu_capability(self.config.memory_pool_size), self.config.memory_pool_size,
                                  compute_dtype=None,
                                  quantize_weights_int8=self.config.enable_quantization and self.config.target_precision == "int8")
        super().__init__(hw, CompilationOptions(target_precision=self.config.target_precision,
                                               compiler_flags=list(self.config.compiler_flags)))
        self.ops = list(hw.get_hardware_capability().supported_operations)


class TpuProvider(CustomProviderAdapter):
    """TPU-style part: bfloat16 compute, one device arena per core summed into the pool."""
    name = "TpuProvider"

    def __init__(self, config: TpuConfig = None):
        self.config = config or TpuConfig()
        pool = min(self.config.core_count * self.config.memory_per_core, 1 << 40)
        hw = HostEmulatedProvider("TpuProvider", tpu_capability(pool), pool,
                                  compute_dtype=torch.bfloat16 if self.config.enable_bfloat16 else None)
        super().__init__(hw, CompilationOptions(target_precision="bf16" if self.config.enable_bfloat16 else "fp32"))
        self.ops = list(hw.get_hardware_capability().supported_operations) + ["AllReduce", "AllGather", "ReduceScatter"]


# ---------------------------------------------------------------------------------------------- WebAssembly target
WASM_PAGE = 64 * 1024


class WasmMemory:
    """Linear memory of the WebAssembly target: grows in 64 KiB pages up to a limit, first-fit allocation with
    coalescing, 16-byte alignment (crates/ronn-providers/src/wasm/allocator.rs:15-247)."""

    def __init__(self, limit_bytes: int, initial_pages: int = 16):
        self.limit_pages = max(limit_bytes // WASM_PAGE, 1)
        self.pages = min(initial_pages, self.limit_pages)
        self._free = [[0, self.pages * WASM_PAGE]]
        self._live: Dict[int, int] = {}
        self.peak_bytes = 0
        self.grow_count = 0

    def _grow(self, need: int) -> bool:
        add = -(-need // WASM_PAGE)
        if self.pages + add > self.limit_pages:
            return False
        start = self.pages * WASM_PAGE
        self.pages += add
        self.grow_count += 1
        if self._free and self._free[-1][0] + self._free[-1][1] == start:
            self._free[-1][1] += add * WASM_PAGE
        else:
            self._free.append([start, add * WASM_PAGE])
        return True

    def allocate(self, size: int) -> int:
        if size <= 0:
            raise ProviderError("allocation size must be positive")
        size = (size + 15) & ~15
        for attempt in range(2):
            for k, (off, sz) in enumerate(self._free):
                if sz >= size:
                    self._free[k:k + 1] = [[off + size, sz - size]] if sz > size else []
                    self._live[off] = size
                    self.peak_bytes = max(self.peak_bytes, sum(self._live.values()))
                    return off
            tail = self._free[-1][1] if self._free and self._free[-1][0] + self._free[-1][1] == self.pages * WASM_PAGE else 0
            if not self._grow(size - tail):
                break
        raise ProviderError(f"WebAssembly memory limit reached: {size} bytes requested, "
                            f"{self.limit_pages * WASM_PAGE - sum(self._live.values())} bytes below the limit")

    def free(self, offset: int) -> None:
        size = self._live.pop(offset, None)
        if size is None:
            raise ProviderError(f"offset {offset} is not allocated")
        self._free.append([offset, size])
        self._free.sort()
        merged = []
        for off, sz in self._free:
            if merged and merged[-1][0] + merged[-1][1] == off:
                merged[-1][1] += sz
            else:
                merged.append([off, sz])
        self._free = merged

    def stats(self) -> Dict[str, int]:
        used = sum(self._live.values())
        return {"pages": self.pages, "limit_pages": self.limit_pages, "allocated_bytes": used, "peak_bytes": self.peak_bytes,
                "free_bytes": self.pages * WASM_PAGE - used, "allocations": len(self._live), "grow_count": self.grow_count}


class WasmModelCache:
    """Compiled-model cache of the WebAssembly target: least recently used first, bounded by total size, entries expire
    (the browser build keeps it in IndexedDB: crates/ronn-providers/src/wasm/bridge.rs:172-305)."""

    def __init__(self, max_bytes: int, expiry_hours: float = 24.0, clock=None):
        import time as _time
        from collections import OrderedDict
        self.max_bytes = max_bytes
        self.expiry_seconds = expiry_hours * 3600.0
        self._clock = clock or _time.time
        self._entries: "OrderedDict[str, tuple]" = OrderedDict()      # key -> (value, size, stored_at)
        self.hits = self.misses = self.evictions = 0

    def put(self, key: str, value, size: int) -> bool:
        if size > self.max_bytes:
            return False
        self._entries.pop(key, None)
        while self._entries and self.total_bytes() + size > self.max_bytes:
            self._entries.popitem(last=False)
            self.evictions += 1
        self._entries[key] = (value, size, self._clock())
        return True

    def get(self, key: str):
        e = self._entries.get(key)
        if e is None or self._clock() - e[2] > self.expiry_seconds:
            if e is not None:
                del self._entries[key]
            self.misses += 1
            return None
        self._entries.move_to_end(key)
        self.hits += 1
        return e[0]

    def total_bytes(self) -> int:
        return sum(e[1] for e in self._entries.values())

    def __len__(self) -> int:
        return len(self._entries)


class WasmProvider(ExecutionProvider):
    provider_id = ProviderType.WASM
    name = "WasmExecutionProvider"
    available = True
    ops = ["Add", "Sub", "Mul", "Div", "MatMul", "Relu", "Sigmoid", "Tanh", "Softmax", "Conv", "MaxPool",
           "AveragePool", "Reshape", "Transpose", "Concat", "Gemm",
           # what the graph optimiser makes of the operators above (MatMul + Add (+ activation), Conv + BN (+ ReLU))
           "FusedGemm", "FusedConv", "Flatten", "Identity", "GlobalAveragePool", "BatchNormalization"]

    def __init__(self, config: WasmProviderConfig = None):
        self.config = config or WasmProviderConfig()
        self.memory = WasmMemory(self.config.memory_limit_bytes)
        self.model_cache = WasmModelCache(self.config.max_cache_size, self.config.cache_expiry_hours) \
            if self.config.enable_model_caching else None

    def get_capability(self) -> ProviderCapability:
        return ProviderCapability(set(self.ops), [DataType.F32, DataType.I32, DataType.U8], [MemoryType.SYSTEM],
                                  PerformanceProfile.POWER_EFFICIENT,
                                  features={"simd128": self.config.enable_simd, "memory_limit": self.config.memory_limit_bytes,
                                            "workers": self.config.worker_count if self.config.enable_web_workers else 0})

    def estimate_performance(self, op_type: str) -> float:
        base = {"Add": 1.0, "Mul": 1.0, "MatMul": 0.6, "Conv": 0.4}.get(op_type, 0.8)
        return base * (1.2 if self.config.enable_simd else 1.0)

    def compile_graph(self, graph, profiler=None):
        """fp32 kernels over the operator registry, restricted to the target's operator list; the constants are
        accounted in the linear memory (a model that does not fit the limit is refused) and compiled models are kept
        in the cache under a key derived from the graph."""
        from ...onnx.registry import default_registry
        unsupported = sorted({n.op_type for n in graph.nodes} - set(self.ops))
        if unsupported:
            raise ProviderError(f"{self.name} does not support operators: {unsupported}")
        key = None
        if self.model_cache is not None:
            import hashlib
            h = hashlib.sha1()
            for n in graph.topological_order():
                h.update(f"{n.op_type}|{n.inputs}|{n.outputs}|{sorted((k, str(v)) for k, v in n.attributes.items())}".encode())
            for name in sorted(graph.initializers):
                t = graph.initializers[name]
                h.update(name.encode() + str(tuple(t.shape)).encode() + t.contiguous().view(torch.uint8).numpy().tobytes()[:4096])
            key = h.hexdigest()
            hit = self.model_cache.get(key)
            if hit is not None:
                return hit
        offsets = []
        try:
            for t in graph.initializers.values():
                if t.numel():
                    offsets.append(self.memory.allocate(t.numel() * 4))
        except ProviderError:
            for o in offsets:
                self.memory.free(o)
            raise
        reg = default_registry()
        kern = build_kernel(graph, torch.device("cpu"), lambda node, g: reg.get(node.op_type).fn,
                            lambda name, t, users: t.float() if t.is_floating_point() else t, self, profiler)
        kern.wasm_offsets = offsets
        if self.model_cache is not None:
            self.model_cache.put(key, kern, sum(t.numel() * 4 for t in graph.initializers.values()))
        return kern

    def release(self, kernel) -> None:
        for o in getattr(kernel, "wasm_offsets", []):
            self.memory.free(o)
        kernel.wasm_offsets = []

"""Providers for targets that do not exist on a B200 box.

The reference ships a browser (WebAssembly) provider and example NPU / TPU providers whose
compile and execute steps are simulated (crates/ronn-providers/src/wasm/provider.rs:23-330,
crates/ronn-providers/src/custom/example_npu.rs:23-389, example_tpu.rs:23-646).  Here they are
registry entries that keep ``ProviderType`` parity, carry the reference's configuration
surface, report ``available = False`` and refuse to compile.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List

from ...api.errors import ProviderError
from ...core.types import (DataType, MemoryType, PerformanceProfile, ProviderCapability, ProviderType)
from ..base import ExecutionProvider


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


class _UnavailableProvider(ExecutionProvider):
    available = False
    ops: List[str] = []
    profile = PerformanceProfile.POWER_EFFICIENT

    def get_capability(self) -> ProviderCapability:
        return ProviderCapability(set(), [DataType.F32], [MemoryType.SYSTEM], self.profile,
                                  features={"available": False, "declared_ops": list(self.ops)})

    def can_handle(self, ops):
        return [False for _ in ops]

    def compile_graph(self, graph, profiler=None):
        raise ProviderError(f"{self.name} is not available on this platform")


class WasmProvider(_UnavailableProvider):
    provider_id = ProviderType.WASM
    name = "WasmExecutionProvider"
    ops = ["Add", "Sub", "Mul", "Div", "MatMul", "Relu", "Sigmoid", "Tanh", "Softmax", "Conv", "MaxPool",
           "AveragePool", "Reshape", "Transpose", "Concat", "Gemm"]

    def __init__(self, config: WasmProviderConfig = None):
        self.config = config or WasmProviderConfig()

    def estimate_performance(self, op_type: str) -> float:
        base = {"Add": 1.0, "Mul": 1.0, "MatMul": 0.6, "Conv": 0.4}.get(op_type, 0.8)
        return base * (1.2 if self.config.enable_simd else 1.0)


class NpuProvider(_UnavailableProvider):
    provider_id = ProviderType.CUSTOM
    name = "NpuProvider"
    ops = ["Conv", "MatMul", "Relu", "MaxPool", "Add"]

    def __init__(self, config: NpuConfig = None):
        self.config = config or NpuConfig()


class TpuProvider(_UnavailableProvider):
    provider_id = ProviderType.CUSTOM
    name = "TpuProvider"
    ops = ["MatMul", "Conv", "AllReduce", "AllGather", "ReduceScatter"]

    def __init__(self, config: TpuConfig = None):
        self.config = config or TpuConfig()

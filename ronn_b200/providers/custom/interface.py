"""Plugin contracts for accelerators this runtime does not know about
(crates/ronn-providers/src/custom/traits.rs:14-330).

A vendor package implements ``CustomHardwareProvider`` (device bring-up, sub-graph compilation, statistics),
``CustomKernel`` (a compiled sub-graph), ``DeviceMemory`` (buffers and copies), and optionally ``HardwareDiscovery`` and
``HardwareProfiler``; ``ProviderPlugin`` is the factory a plugin module exports.  ``CustomProviderAdapter`` turns any
such provider into an ``ExecutionProvider`` so that ``Model.create_session`` can run a graph on it.
"""
from __future__ import annotations

import enum
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ...api.errors import ProviderError
from ...core.types import (DataType, KernelStats, MemoryType, MemoryUsage, PerformanceProfile, ProviderCapability,
                           ProviderType)
from ...graph.ir import ModelGraph, SubGraph
from ..base import ExecutionProvider

ABI_VERSION = 1


@dataclass
class PowerProfile:
    idle_power_watts: float = 0.0
    peak_power_watts: float = 0.0
    tdp_watts: float = 0.0
    efficiency_tops_per_watt: float = 0.0


@dataclass
class HardwareCapability:
    vendor: str
    model: str
    architecture_version: str = ""
    supported_data_types: List[DataType] = field(default_factory=lambda: [DataType.F32])
    max_memory_bytes: int = 0
    peak_tops: float = 0.0
    memory_bandwidth_gbps: float = 0.0
    supported_operations: List[str] = field(default_factory=list)
    features: Dict[str, str] = field(default_factory=dict)
    power_profile: PowerProfile = field(default_factory=PowerProfile)


@dataclass
class ProviderStats:
    total_operations: int = 0
    average_execution_time_us: float = 0.0
    memory_usage_bytes: int = 0
    peak_memory_bytes: int = 0
    hardware_utilization: float = 0.0
    current_power_watts: float = 0.0
    total_energy_joules: float = 0.0


@dataclass
class KernelInfo:
    name: str
    operations: List[str]
    estimated_memory_bytes: int = 0
    estimated_execution_time_us: float = 0.0
    hardware_utilization: float = 0.0
    compilation_time_ms: float = 0.0


@dataclass
class DeviceBuffer:
    handle: int
    size: int
    alignment: int
    device_id: int = 0
    memory_type: str = "device"


@dataclass
class DeviceMemoryInfo:
    total_bytes: int
    available_bytes: int
    allocated_bytes: int
    bandwidth_gbps: float = 0.0
    memory_type: str = "device"


@dataclass
class CompilationOptions:
    optimization_level: int = 2
    aggressive_optimization: bool = False
    target_precision: str = "fp32"
    compiler_flags: List[str] = field(default_factory=list)
    defines: Dict[str, str] = field(default_factory=dict)
    include_paths: List[str] = field(default_factory=list)


class DeviceStatus(enum.Enum):
    AVAILABLE = "available"
    BUSY = "busy"
    ERROR = "error"
    NOT_INITIALIZED = "not_initialized"
    OFFLINE = "offline"


@dataclass
class HardwareDevice:
    device_id: str
    name: str
    vendor: str
    device_type: str
    capabilities: HardwareCapability
    driver_version: str = ""
    firmware_version: str = ""
    status: DeviceStatus = DeviceStatus.AVAILABLE
    error: Optional[str] = None


@dataclass
class ProfilingSession:
    session_id: int
    operation_name: str
    start_time: float


@dataclass
class ProfilingResults:
    operation_name: str
    execution_time_us: float
    memory_usage_bytes: int = 0
    hardware_utilization: float = 0.0
    power_consumption_watts: float = 0.0
    energy_consumed_mj: float = 0.0
    custom_metrics: Dict[str, float] = field(default_factory=dict)


@dataclass
class ProfilingSummary:
    total_operations: int = 0
    total_execution_time_us: float = 0.0
    average_execution_time_us: float = 0.0
    peak_memory_bytes: int = 0
    average_utilization: float = 0.0
    total_energy_joules: float = 0.0
    top_operations_by_time: List[Tuple[str, float]] = field(default_factory=list)


class DeviceMemory(ABC):
    @abstractmethod
    def allocate(self, size: int, alignment: int = 64) -> DeviceBuffer: ...

    @abstractmethod
    def deallocate(self, buffer: DeviceBuffer) -> None: ...

    @abstractmethod
    def copy_to_device(self, host_data: bytes, buffer: DeviceBuffer) -> None: ...

    @abstractmethod
    def copy_from_device(self, buffer: DeviceBuffer, nbytes: Optional[int] = None) -> bytes: ...

    @abstractmethod
    def get_memory_info(self) -> DeviceMemoryInfo: ...

    def synchronize(self) -> None:
        pass

    def can_access(self, a: DeviceBuffer, b: DeviceBuffer) -> bool:
        return a.device_id == b.device_id


class CustomKernel(ABC):
    @abstractmethod
    def execute(self, inputs: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]: ...

    @abstractmethod
    def get_memory_usage(self) -> MemoryUsage: ...

    @abstractmethod
    def get_performance_stats(self) -> KernelStats: ...

    @abstractmethod
    def get_kernel_info(self) -> KernelInfo: ...

    def warmup(self) -> None:
        pass


class CustomHardwareProvider(ABC):
    @abstractmethod
    def provider_name(self) -> str: ...

    @abstractmethod
    def get_hardware_capability(self) -> HardwareCapability: ...

    @abstractmethod
    def is_hardware_available(self) -> bool: ...

    @abstractmethod
    def initialize(self) -> None: ...

    @abstractmethod
    def compile_subgraph(self, subgraph: SubGraph, initializers: Optional[Dict[str, torch.Tensor]] = None,
                         options: Optional[CompilationOptions] = None) -> CustomKernel: ...

    @abstractmethod
    def get_device_memory(self) -> DeviceMemory: ...

    @abstractmethod
    def get_performance_stats(self) -> ProviderStats: ...

    @abstractmethod
    def shutdown(self) -> None: ...


class HardwareDiscovery(ABC):
    @abstractmethod
    def discover_devices(self) -> List[HardwareDevice]: ...

    def is_device_available(self, device_id: str) -> bool:
        d = self.get_device_info(device_id)
        return d is not None and d.status == DeviceStatus.AVAILABLE

    def get_device_info(self, device_id: str) -> Optional[HardwareDevice]:
        return next((d for d in self.discover_devices() if d.device_id == device_id), None)


class HardwareProfiler(ABC):
    @abstractmethod
    def start_profiling(self, operation_name: str) -> ProfilingSession: ...

    @abstractmethod
    def stop_profiling(self, session: ProfilingSession) -> ProfilingResults: ...

    @abstractmethod
    def get_profiling_summary(self) -> ProfilingSummary: ...

    @abstractmethod
    def reset_profiling(self) -> None: ...


class WallClockProfiler(HardwareProfiler):
    """Profiler that any provider can use: wall-clock time per named operation, energy from a constant power draw."""

    def __init__(self, power_watts: float = 0.0):
        self.power_watts = power_watts
        self._next = 1
        self._open: Dict[int, ProfilingSession] = {}
        self._by_op: Dict[str, List[float]] = {}
        self._peak_mem = 0
        self._util: List[float] = []

    def start_profiling(self, operation_name: str) -> ProfilingSession:
        s = ProfilingSession(self._next, operation_name, time.perf_counter())
        self._next += 1
        self._open[s.session_id] = s
        return s

    def stop_profiling(self, session: ProfilingSession, memory_usage_bytes: int = 0, hardware_utilization: float = 0.0,
                       **custom) -> ProfilingResults:
        if self._open.pop(session.session_id, None) is None:
            raise ProviderError(f"profiling session {session.session_id} is not open")
        us = (time.perf_counter() - session.start_time) * 1e6
        self._by_op.setdefault(session.operation_name, []).append(us)
        self._peak_mem = max(self._peak_mem, memory_usage_bytes)
        self._util.append(hardware_utilization)
        return ProfilingResults(session.operation_name, us, memory_usage_bytes, hardware_utilization, self.power_watts,
                                self.power_watts * us * 1e-3, {k: float(v) for k, v in custom.items()})

    def get_profiling_summary(self) -> ProfilingSummary:
        n = sum(len(v) for v in self._by_op.values())
        total = sum(sum(v) for v in self._by_op.values())
        top = sorted(((k, sum(v)) for k, v in self._by_op.items()), key=lambda kv: -kv[1])[:10]
        return ProfilingSummary(n, total, total / n if n else 0.0, self._peak_mem,
                                sum(self._util) / len(self._util) if self._util else 0.0,
                                self.power_watts * total * 1e-6, top)

    def reset_profiling(self) -> None:
        self._open.clear()
        self._by_op.clear()
        self._util.clear()
        self._peak_mem = 0


@dataclass
class PluginMetadata:
    name: str
    version: str = "0.0.0"
    author: str = ""
    description: str = ""
    license: str = ""
    min_ronn_version: str = "0.1.0"
    supported_hardware: List[str] = field(default_factory=list)
    abi_version: int = ABI_VERSION
    plugin_path: str = ""
    status: str = "loaded"            # loaded | load_error:<why> | disabled | incompatible


class ProviderPlugin(ABC):
    """What a plugin module exports through ``ronn_plugin()``."""

    @abstractmethod
    def get_metadata(self) -> PluginMetadata: ...

    @abstractmethod
    def create_provider(self, config: Optional[dict] = None) -> CustomHardwareProvider: ...

    @abstractmethod
    def is_hardware_available(self) -> bool: ...

    def get_abi_version(self) -> int:
        return ABI_VERSION


class _AdapterKernel:
    """CompiledKernel face of a CustomKernel (what ``InferenceSession`` calls)."""

    def __init__(self, kernel: CustomKernel):
        self.kernel = kernel
        self.stats = kernel.get_performance_stats()
        self.device = torch.device("cpu")       # tensors cross the session boundary in host memory
        self.profiler = None

    def execute(self, inputs: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return self.kernel.execute(inputs)

    def get_memory_usage(self) -> MemoryUsage:
        return self.kernel.get_memory_usage()

    def get_performance_stats(self) -> KernelStats:
        return self.kernel.get_performance_stats()


class CustomProviderAdapter(ExecutionProvider):
    """Presents a ``CustomHardwareProvider`` to the session / provider registry as ``ProviderType.CUSTOM``."""
    provider_id = ProviderType.CUSTOM

    def __init__(self, provider: CustomHardwareProvider, options: Optional[CompilationOptions] = None):
        if not provider.is_hardware_available():
            raise ProviderError(f"{provider.provider_name()}: hardware is not available")
        self.provider = provider
        self.options = options or CompilationOptions()
        self.name = provider.provider_name()
        provider.initialize()

    def get_capability(self) -> ProviderCapability:
        cap = self.provider.get_hardware_capability()
        return ProviderCapability(set(cap.supported_operations), list(cap.supported_data_types), [MemoryType.DEVICE],
                                  PerformanceProfile.POWER_EFFICIENT,
                                  features={"vendor": cap.vendor, "model": cap.model, **cap.features})

    def compile_graph(self, graph: ModelGraph, profiler=None):
        sub = SubGraph(list(graph.topological_order()), [], [i.name for i in graph.inputs], [o.name for o in graph.outputs])
        unsupported = sorted({n.op_type for n in sub.nodes} - set(self.provider.get_hardware_capability().supported_operations))
        if unsupported:
            raise ProviderError(f"{self.name} does not support operators: {unsupported}")
        return _AdapterKernel(self.provider.compile_subgraph(sub, dict(graph.initializers), self.options))

    def shutdown(self) -> None:
        self.provider.shutdown()

"""Core type system.

Mirrors the reference's enums and provider contracts
(crates/ronn-core/src/types.rs:24-35 DataType, :39-60 ProviderId, :77-82 TensorLayout,
:86-103 AttributeValue, :217-229 ProviderCapability, :269-279 ProviderConfig,
:294-333 allocator structs) with exactly one OptimizationLevel (O0-O3; the reference
has two: types.rs:282-292 and crates/ronn-graph/src/optimizer.rs:8-18).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


class DataType(enum.Enum):
    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"
    I8 = "i8"
    I32 = "i32"
    I64 = "i64"
    U8 = "u8"
    U32 = "u32"
    BOOL = "bool"
    F64 = "f64"

    @property
    def torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @property
    def itemsize(self) -> int:
        return {DataType.F32: 4, DataType.F16: 2, DataType.BF16: 2, DataType.I8: 1, DataType.I32: 4,
                DataType.I64: 8, DataType.U8: 1, DataType.U32: 4, DataType.BOOL: 1, DataType.F64: 8}[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DataType":
        for k, v in _TO_TORCH.items():
            if v == dt:
                return k
        raise TypeError(f"unsupported torch dtype {dt}")


_TO_TORCH = {
    DataType.F32: torch.float32, DataType.F16: torch.float16, DataType.BF16: torch.bfloat16,
    DataType.I8: torch.int8, DataType.I32: torch.int32, DataType.I64: torch.int64,
    DataType.U8: torch.uint8, DataType.U32: torch.uint32, DataType.BOOL: torch.bool,
    DataType.F64: torch.float64,
}


class ProviderType(enum.Enum):
    """Execution providers selectable on a session (crates/ronn-core/src/types.rs:39-60)."""
    CPU = "cpu"
    GPU = "gpu"
    BITNET = "bitnet"
    WASM = "wasm"
    CUSTOM = "custom"

    @staticmethod
    def parse(s) -> "ProviderType":
        if isinstance(s, ProviderType):
            return s
        key = str(s).strip().lower()
        alias = {"cpu": ProviderType.CPU, "gpu": ProviderType.GPU, "cuda": ProviderType.GPU,
                 "bitnet": ProviderType.BITNET, "wasm": ProviderType.WASM, "webassembly": ProviderType.WASM,
                 "custom": ProviderType.CUSTOM}
        if key not in alias:
            raise ValueError(f"unknown provider '{s}' (expected cpu|gpu|cuda|bitnet|wasm)")
        return alias[key]


ProviderId = ProviderType


class OptimizationLevel(enum.IntEnum):
    """O0 none; O1 constant folding + DCE; O2 + fusion + layout; O3 + provider-specific passes."""
    O0 = 0
    O1 = 1
    O2 = 2
    O3 = 3

    @staticmethod
    def parse(s) -> "OptimizationLevel":
        if isinstance(s, OptimizationLevel):
            return s
        if isinstance(s, int):
            return OptimizationLevel(s)
        key = str(s).strip().lower()
        alias = {"o0": 0, "none": 0, "o1": 1, "basic": 1, "o2": 2, "default": 2, "o3": 3, "aggressive": 3}
        if key not in alias:
            raise ValueError(f"unknown optimization level '{s}' (expected O0..O3|none|basic|default|aggressive)")
        return OptimizationLevel(alias[key])


class TensorLayout(enum.Enum):
    ROW_MAJOR = "row_major"
    COLUMN_MAJOR = "column_major"


class MemoryType(enum.Enum):
    SYSTEM = "system"
    DEVICE = "device"
    SHARED = "shared"
    PINNED = "pinned"


class PerformanceProfile(enum.Enum):
    CPU = "cpu"
    GPU = "gpu"
    MEMORY_OPTIMIZED = "memory_optimized"
    POWER_EFFICIENT = "power_efficient"


@dataclass
class OperatorSpec:
    op_type: str
    input_types: List[DataType] = field(default_factory=list)
    output_types: List[DataType] = field(default_factory=list)
    attributes: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ResourceRequirements:
    min_memory_bytes: Optional[int] = None
    cpu_features: List[str] = field(default_factory=list)
    gpu_memory_bytes: Optional[int] = None


@dataclass
class ProviderCapability:
    supported_ops: set
    data_types: List[DataType]
    memory_types: List[MemoryType]
    performance_profile: PerformanceProfile
    resource_requirements: ResourceRequirements = field(default_factory=ResourceRequirements)
    features: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ProviderConfig:
    thread_count: Optional[int] = None
    memory_limit: Optional[int] = None
    optimization_level: OptimizationLevel = OptimizationLevel.O2
    custom_options: Dict[str, str] = field(default_factory=dict)


@dataclass
class TensorBuffer:
    ptr: int
    size: int
    alignment: int
    memory_type: MemoryType


@dataclass
class MemoryInfo:
    total_bytes: int
    allocated_bytes: int
    peak_bytes: int


@dataclass
class KernelStats:
    execution_count: int = 0
    average_time_us: float = 0.0
    min_time_us: float = 0.0
    max_time_us: float = 0.0

    def record(self, us: float) -> None:
        n = self.execution_count
        self.average_time_us = (self.average_time_us * n + us) / (n + 1)
        self.min_time_us = us if n == 0 else min(self.min_time_us, us)
        self.max_time_us = max(self.max_time_us, us)
        self.execution_count = n + 1


@dataclass
class MemoryUsage:
    peak_bytes: int = 0
    current_bytes: int = 0
    allocation_count: int = 0

"""A custom-hardware provider that is real and runs anywhere: the "device" is a byte arena in host memory.

It is the reference implementation of the plugin contracts (``interface.py``): a vendor copies its shape.  The memory
manager hands out aligned, bounds-checked buffers from a fixed arena (first fit, coalescing free list) and enforces
the device's memory limit; kernels are sub-graphs compiled over the CPU operator registry whose constant tensors are
staged through device buffers, with an optional numeric personality (int8 weight quantisation for an NPU-like part,
bfloat16 compute for a TPU-like part).  The reference's NPU / TPU examples simulate their devices with sleeps
(crates/ronn-providers/src/custom/example_npu.rs:23-389, example_tpu.rs:23-646); these compute the actual results.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch

from ...api.errors import ProviderError
from ...core.types import DataType, KernelStats, MemoryUsage
from ...graph.ir import ModelGraph, SubGraph, TensorInfo
from ..base import build_kernel
from .interface import (CompilationOptions, CustomHardwareProvider, CustomKernel, DeviceBuffer, DeviceMemory,
                        DeviceMemoryInfo, DeviceStatus, HardwareCapability, HardwareDevice, HardwareDiscovery,
                        KernelInfo, PowerProfile, ProviderStats, WallClockProfiler)


class ArenaMemory(DeviceMemory):
    """First-fit allocator over one contiguous arena; handles are offsets, every access is bounds-checked."""

    def __init__(self, total_bytes: int, device_id: int = 0, bandwidth_gbps: float = 0.0, memory_type: str = "device"):
        if total_bytes <= 0:
            raise ProviderError("device memory size must be positive")
        self.total = int(total_bytes)
        self.device_id = device_id
        self.bandwidth = bandwidth_gbps
        self.memory_type = memory_type
        self._arena = bytearray()                              # grows to the highest offset handed out so far
        self._free: List[List[int]] = [[0, self.total]]          # [offset, size], sorted by offset
        self._live: Dict[int, int] = {}                          # handle -> size
        self._lock = threading.Lock()
        self.peak = 0

    def allocate(self, size: int, alignment: int = 64) -> DeviceBuffer:
        if size <= 0:
            raise ProviderError("allocation size must be positive")
        if alignment <= 0 or alignment & (alignment - 1):
            raise ProviderError("alignment must be a power of two")
        with self._lock:
            for k, (off, sz) in enumerate(self._free):
                start = (off + alignment - 1) & ~(alignment - 1)
                pad = start - off
                if sz >= pad + size:
                    rest = sz - pad - size
                    pieces = ([[off, pad]] if pad else []) + ([[start + size, rest]] if rest else [])
                    self._free[k:k + 1] = pieces
                    self._live[start] = size
                    if len(self._arena) < start + size:
                        self._arena.extend(bytes(start + size - len(self._arena)))
                    used = sum(self._live.values())
                    self.peak = max(self.peak, used)
                    return DeviceBuffer(start, size, alignment, self.device_id, self.memory_type)
        raise ProviderError(f"out of device memory: {size} bytes requested, {self.get_memory_info().available_bytes} free")

    def deallocate(self, buffer: DeviceBuffer) -> None:
        with self._lock:
            size = self._live.pop(buffer.handle, None)
            if size is None:
                raise ProviderError(f"buffer {buffer.handle} is not allocated on this device")
            self._free.append([buffer.handle, size])
            self._free.sort()
            merged: List[List[int]] = []
            for off, sz in self._free:
                if merged and merged[-1][0] + merged[-1][1] == off:
                    merged[-1][1] += sz
                else:
                    merged.append([off, sz])
            self._free = merged

    def _check(self, buffer: DeviceBuffer, nbytes: int) -> None:
        if buffer.device_id != self.device_id or self._live.get(buffer.handle) != buffer.size:
            raise ProviderError("buffer does not belong to this device")
        if nbytes < 0 or nbytes > buffer.size:
            raise ProviderError(f"copy of {nbytes} bytes exceeds the {buffer.size}-byte buffer")

    def copy_to_device(self, host_data: bytes, buffer: DeviceBuffer) -> None:
        n = len(host_data)
        self._check(buffer, n)
        self._arena[buffer.handle: buffer.handle + n] = host_data

    def copy_from_device(self, buffer: DeviceBuffer, nbytes: Optional[int] = None) -> bytes:
        n = buffer.size if nbytes is None else nbytes
        self._check(buffer, n)
        return bytes(self._arena[buffer.handle: buffer.handle + n])

    def view(self, buffer: DeviceBuffer) -> memoryview:
        self._check(buffer, buffer.size)
        return memoryview(self._arena)[buffer.handle: buffer.handle + buffer.size]

    def get_memory_info(self) -> DeviceMemoryInfo:
        used = sum(self._live.values())
        return DeviceMemoryInfo(self.total, self.total - used, used, self.bandwidth, self.memory_type)


class HostKernel(CustomKernel):
    def __init__(self, name: str, graph: ModelGraph, kernel, buffers: List[DeviceBuffer], memory: ArenaMemory,
                 provider: "HostEmulatedProvider", compile_ms: float):
        self.name, self.graph, self._kernel, self._buffers = name, graph, kernel, buffers
        self._memory, self._provider, self._compile_ms = memory, provider, compile_ms
        self._const_bytes = sum(b.size for b in buffers)
        self.stats = KernelStats()

    def execute(self, inputs: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        prof = self._provider.profiler
        sess = prof.start_profiling(self.name)
        t0 = time.perf_counter()
        cast = self._provider.compute_dtype
        feeds = {k: (v.to(cast) if cast is not None and v.is_floating_point() else v) for k, v in inputs.items()}
        out = self._kernel.execute(feeds)
        out = {k: (v.float() if cast is not None and v.is_floating_point() else v) for k, v in out.items()}
        us = (time.perf_counter() - t0) * 1e6
        self.stats.record(us)
        prof.stop_profiling(sess, memory_usage_bytes=self._const_bytes)
        self._provider._record(us)
        return out

    def get_memory_usage(self) -> MemoryUsage:
        return MemoryUsage(self._const_bytes, self._const_bytes, len(self._buffers))

    def get_performance_stats(self) -> KernelStats:
        return self.stats

    def get_kernel_info(self) -> KernelInfo:
        return KernelInfo(self.name, [n.op_type for n in self.graph.nodes], self._const_bytes,
                          self.stats.average_time_us, 0.0, self._compile_ms)

    def release(self) -> None:
        for b in self._buffers:
            self._memory.deallocate(b)
        self._buffers = []


class HostEmulatedProvider(CustomHardwareProvider):
    """Executes sub-graphs on the host with the accelerator's numeric personality; constants live in device buffers."""

    def __init__(self, name: str, capability: HardwareCapability, memory_bytes: int, compute_dtype: Optional[torch.dtype] = None,
                 quantize_weights_int8: bool = False, device_id: int = 0):
        self._name = name
        self._cap = capability
        self.compute_dtype = compute_dtype
        self.quantize_weights_int8 = quantize_weights_int8
        self.memory = ArenaMemory(memory_bytes, device_id, capability.memory_bandwidth_gbps)
        self.profiler = WallClockProfiler(capability.power_profile.tdp_watts)
        self._initialized = False
        self._kernels: List[HostKernel] = []
        self._ops = 0
        self._total_us = 0.0

    def provider_name(self) -> str:
        return self._name

    def get_hardware_capability(self) -> HardwareCapability:
        return self._cap

    def is_hardware_available(self) -> bool:
        return True

    def initialize(self) -> None:
        self._initialized = True

    def get_device_memory(self) -> DeviceMemory:
        return self.memory

    def _record(self, us: float) -> None:
        self._ops += 1
        self._total_us += us

    def _stage_constant(self, t: torch.Tensor, quantize: bool, buffers: List[DeviceBuffer]) -> torch.Tensor:
        """Round-trips a constant through device memory (what a real driver upload does), applying the part's weight
        format on the way: symmetric per-tensor int8 for an NPU-like part, the compute dtype otherwise."""
        if quantize and t.is_floating_point() and t.dim() >= 2:
            scale = float(t.abs().max().clamp_min(1e-12)) / 127.0
            q = torch.clamp(torch.round(t.float() / scale), -127, 127).to(torch.int8).contiguous()
            buf = self.memory.allocate(q.numel(), 64)
            self.memory.copy_to_device(q.numpy().tobytes(), buf)
            buffers.append(buf)
            back = torch.frombuffer(bytearray(self.memory.copy_from_device(buf)), dtype=torch.int8).reshape(q.shape)
            w = back.float() * scale
            return w.to(self.compute_dtype) if self.compute_dtype is not None else w.to(t.dtype)
        src = t.to(self.compute_dtype) if (self.compute_dtype is not None and t.is_floating_point()) else t
        src = src.contiguous()
        raw = src.view(torch.uint8).reshape(-1) if src.numel() else src.reshape(-1).view(torch.uint8)
        if raw.numel() == 0:
            return src
        buf = self.memory.allocate(raw.numel(), 64)
        self.memory.copy_to_device(raw.numpy().tobytes(), buf)
        buffers.append(buf)
        back = torch.frombuffer(bytearray(self.memory.copy_from_device(buf)), dtype=torch.uint8)
        return back.view(src.dtype).reshape(src.shape)

    def compile_subgraph(self, subgraph: SubGraph, initializers=None, options: Optional[CompilationOptions] = None) -> CustomKernel:
        if not self._initialized:
            raise ProviderError(f"{self._name} is not initialised")
        if not subgraph.nodes:
            raise ProviderError("cannot compile an empty subgraph")
        unsupported = sorted({n.op_type for n in subgraph.nodes} - set(self._cap.supported_operations))
        if unsupported:
            raise ProviderError(f"{self._name} does not support operators: {unsupported}")
        from ...onnx.registry import default_registry
        t0 = time.perf_counter()
        g = ModelGraph.from_nodes([n.clone() for n in subgraph.nodes])
        buffers: List[DeviceBuffer] = []
        try:
            weight_inputs = {n.inputs[1] for n in g.nodes if n.op_type in ("MatMul", "Gemm", "Conv", "FusedGemm", "FusedConv")
                             and len(n.inputs) > 1}
            g.initializers = {k: self._stage_constant(v, self.quantize_weights_int8 and k in weight_inputs, buffers)
                              for k, v in (initializers or {}).items()}
            g.inputs = [TensorInfo(i, [], DataType.F32) for i in subgraph.inputs if i not in g.initializers]
            g.outputs = [TensorInfo(o, [], DataType.F32) for o in subgraph.outputs]
            reg = default_registry()
            kern = build_kernel(g, torch.device("cpu"), lambda node, gg: reg.get(node.op_type).fn, lambda n, t, u: t, None, None)
        except Exception:
            for b in buffers:
                self.memory.deallocate(b)
            raise
        k = HostKernel(f"{self._name}_kernel_{len(self._kernels)}", g, kern, buffers, self.memory, self,
                       (time.perf_counter() - t0) * 1e3)
        self._kernels.append(k)
        return k

    def get_performance_stats(self) -> ProviderStats:
        info = self.memory.get_memory_info()
        tdp = self._cap.power_profile.tdp_watts
        return ProviderStats(self._ops, self._total_us / self._ops if self._ops else 0.0, info.allocated_bytes,
                             self.memory.peak, 0.0, tdp if self._ops else self._cap.power_profile.idle_power_watts,
                             tdp * self._total_us * 1e-6)

    def shutdown(self) -> None:
        for k in self._kernels:
            k.release()
        self._kernels = []
        self._initialized = False


class StaticDiscovery(HardwareDiscovery):
    """Discovery over a fixed list of devices (what a plugin that probed its driver at import time would return)."""

    def __init__(self, devices: List[HardwareDevice]):
        self._devices = list(devices)

    def discover_devices(self) -> List[HardwareDevice]:
        return list(self._devices)

    def set_status(self, device_id: str, status: DeviceStatus, error: Optional[str] = None) -> None:
        for d in self._devices:
            if d.device_id == device_id:
                d.status, d.error = status, error


_NPU_OPS = ["Conv", "MatMul", "Gemm", "Relu", "MaxPool", "AveragePool", "GlobalAveragePool", "Add", "Mul", "Sigmoid",
            "Softmax", "Flatten", "Reshape", "BatchNormalization", "FusedConv", "FusedGemm", "Clip", "Concat"]
_TPU_OPS = ["MatMul", "Gemm", "Conv", "Add", "Mul", "Sub", "Relu", "Gelu", "Tanh", "Softmax", "LayerNormalization",
            "Transpose", "Reshape", "Attention", "FusedGemm", "Concat", "Split", "Gather", "ReduceMean", "Erf", "Sqrt",
            "Div", "Pow", "Flatten"]


def npu_capability(memory_bytes: int = 2 << 30) -> HardwareCapability:
    return HardwareCapability("ronn", "host-emulated NPU", "1", [DataType.F32, DataType.I8, DataType.U8], memory_bytes, 26.0,
                              68.0, list(_NPU_OPS), {"weights": "int8 symmetric per tensor", "activations": "fp32"},
                              PowerProfile(0.5, 8.0, 5.0, 5.2))


def tpu_capability(memory_bytes: int = 8 << 30) -> HardwareCapability:
    return HardwareCapability("ronn", "host-emulated TPU", "v4", [DataType.BF16, DataType.F32], memory_bytes, 275.0, 1200.0,
                              list(_TPU_OPS), {"compute": "bfloat16", "matrix_unit": "128x128"},
                              PowerProfile(60.0, 192.0, 170.0, 1.6))

"""BitNet execution provider (crates/ronn-providers/src/bitnet/provider.rs:25-386).

Declares the reference's twelve operators and its speed-up constants; MatMul / Gemm nodes whose
weight is an initializer are compiled to 1-bit or ternary kernels (weights quantised once at
compile time - the reference re-quantises both operands on every call, bitnet/kernels.rs:265-278),
``com.ronn::BitLinear`` nodes run the packed ternary x int8 kernel, everything else uses the
full-precision operator table.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ...core.types import (DataType, MemoryType, PerformanceProfile, ProviderCapability, ProviderConfig, ProviderType)
from ...graph.ir import ModelGraph
from ...onnx.registry import default_registry
from ..allocator import BitNetAllocator
from ..base import CompiledKernel, ExecutionProvider, build_kernel
from .quantization import QuantizationMethod, pack_ternary_rows, quantize_binary, quantize_ternary

BITNET_OPS = ["MatMul", "Gemm", "Conv", "Add", "Sub", "Mul", "And", "Or", "Xor", "BatchNormalization", "Relu", "Sigmoid"]


@dataclass
class BitNetProviderConfig:
    quantization_method: QuantizationMethod = QuantizationMethod.BINARY
    enable_kernel_caching: bool = True
    max_cache_size: int = 64 * 1024 * 1024
    enable_mixed_precision: bool = True
    memory_optimization_level: int = 2
    enable_simd: bool = True


class BitNetExecutionProvider(ExecutionProvider):
    provider_id = ProviderType.BITNET
    name = "BitNetExecutionProvider"

    def __init__(self, config: BitNetProviderConfig = None):
        self.config = config or BitNetProviderConfig()
        self.allocator = BitNetAllocator()

    def estimate_speedup(self, op_type: str) -> float:
        m = self.config.quantization_method
        table = {"MatMul": {QuantizationMethod.BINARY: 64.0, QuantizationMethod.TERNARY: 32.0, QuantizationMethod.ASYMMETRIC: 48.0},
                 "Gemm": {QuantizationMethod.BINARY: 64.0, QuantizationMethod.TERNARY: 32.0, QuantizationMethod.ASYMMETRIC: 48.0},
                 "Conv": {QuantizationMethod.BINARY: 32.0, QuantizationMethod.TERNARY: 24.0, QuantizationMethod.ASYMMETRIC: 28.0}}
        if op_type in table:
            return table[op_type][m]
        if op_type in ("And", "Or", "Xor"):
            return 128.0
        if op_type in ("Add", "Sub", "Mul", "Relu", "Sigmoid"):
            return 16.0
        return 1.0

    def get_capability(self) -> ProviderCapability:
        return ProviderCapability(
            supported_ops=set(default_registry().supported_ops()),
            data_types=[DataType.F32, DataType.BF16, DataType.F16, DataType.I8, DataType.U8, DataType.BOOL],
            memory_types=[MemoryType.SYSTEM, MemoryType.DEVICE],
            performance_profile=PerformanceProfile.MEMORY_OPTIMIZED,
            features={"quantization": self.config.quantization_method.value, "native_ops": list(BITNET_OPS)})

    def configure(self, config: ProviderConfig) -> None:
        opts = config.custom_options
        if "quantization_method" in opts:
            self.config.quantization_method = QuantizationMethod(opts["quantization_method"].lower())
        if "enable_simd" in opts:
            self.config.enable_simd = opts["enable_simd"].lower() in ("1", "true", "yes")

    def get_allocator(self):
        return self.allocator

    def compile_graph(self, graph: ModelGraph, profiler=None) -> CompiledKernel:
        reg = default_registry()
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        method = self.config.quantization_method
        quantized = {}

        def quant_weight(name):
            if name not in quantized:
                w = graph.initializers[name].float()
                if method == QuantizationMethod.BINARY:
                    q = quantize_binary(w)
                else:
                    q = quantize_ternary(w, "absmean" if method == QuantizationMethod.ASYMMETRIC else "threshold")
                quantized[name] = q.dequantize().to(dev)
            return quantized[name]

        def resolve(node, g):
            if node.op_type in ("MatMul", "Gemm", "FusedGemm") and len(node.inputs) > 1 \
                    and node.inputs[1] in g.initializers and g.initializers[node.inputs[1]].dim() == 2 \
                    and g.initializers[node.inputs[1]].is_floating_point():
                wq = quant_weight(node.inputs[1])
                inner = reg.get(node.op_type).fn

                def run(i, a, c, _w=wq, _f=inner):
                    i = list(i)
                    i[1] = _w.to(i[0].dtype)
                    return _f(i, a, c)
                return run
            return reg.get(node.op_type).fn

        def place(name, t, users):
            return t.to(dev)

        return build_kernel(graph, dev, resolve, place, self, profiler)

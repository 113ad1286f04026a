"""CPU execution provider (crates/ronn-providers/src/cpu/provider.rs:25-375,
crates/ronn-providers/src/cpu/kernels.rs:20-478).

Nodes resolve to the operator registry on CPU tensors; small fp32 GEMMs tagged by the CPU
optimisation pass run on the native AVX2/AVX-512 kernel, which is where the batch-1 MLP
spends its time once per-node dispatch is a table lookup.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .. import _native
from ..api.errors import ProviderError
from ..core.types import (DataType, MemoryType, PerformanceProfile, ProviderCapability, ProviderConfig, ProviderType,
                          ResourceRequirements)
from ..graph.ir import ModelGraph
from ..onnx.registry import default_registry
from .allocator import PooledMemoryAllocator
from .base import CompiledKernel, ExecutionProvider, build_kernel


def detect_simd_features():
    lvl = _native.host().ronn_cpu_simd_level()
    feats = []
    if lvl >= 1:
        feats += ["avx2", "fma"]
    if lvl >= 2:
        feats += ["avx512f"]
    return feats


def _simd_gemm(inputs, attrs, ctx):
    x, w = inputs[0], inputs[1]
    bias = inputs[2] if len(inputs) > 2 else None
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or x.device.type != "cpu":
        return default_registry().get("FusedGemm").fn(inputs, attrs, ctx)
    M, K = x.shape
    N = w.shape[1]
    out = torch.empty((M, N), dtype=torch.float32)
    act = 1 if attrs.get("activation", "") == "Relu" else 0
    _native.host().ronn_cpu_gemm_f32(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                     out.data_ptr(), M, N, K, act)
    return [out]


class ChainKernel:
    """A linear fp32 chain of dense layers / ReLU / final softmax executed by ONE native call
    (the fused forms the reference names but never produces: crates/ronn-providers/src/cpu/kernels.rs:20-31)."""

    def __init__(self, graph: ModelGraph, order):
        import ctypes as C
        import numpy as np
        from ..core.types import KernelStats
        self.device = torch.device("cpu")
        self.input_name = graph.inputs[0].name
        self.output_name = graph.outputs[0].name
        self.stats = KernelStats()
        self.steps = order
        kinds, acts, dims, self._keep = [], [], [], []
        wptr, bptr = [], []
        k0 = None
        for n in order:
            if n.op_type in ("FusedGemm", "MatMul", "Gemm"):
                w = graph.initializers[n.inputs[1]].contiguous()
                b = graph.initializers[n.inputs[2]].contiguous() if len(n.inputs) > 2 and n.inputs[2] else None
                self._keep += [w, b]
                if k0 is None:
                    k0 = w.shape[0]
                kinds.append(0)
                acts.append(1 if n.attr("activation", "") == "Relu" else 0)
                dims.append(w.shape[1])
                wptr.append(w.data_ptr())
                bptr.append(b.data_ptr() if b is not None else None)
            else:
                kinds.append(1 if n.op_type == "Relu" else 2)
                acts.append(0)
                dims.append(dims[-1] if dims else 0)
                wptr.append(None)
                bptr.append(None)
        self.k0, self.n_out, self.max_n = k0, dims[-1], max(dims)
        n = len(kinds)
        self._kinds = (C.c_int32 * n)(*kinds)
        self._acts = (C.c_int32 * n)(*acts)
        self._dims = (C.c_int64 * n)(*dims)
        self._w = (C.c_void_p * n)(*wptr)
        self._b = (C.c_void_p * n)(*bptr)
        self._n = n
        self._fn = _native.host().ronn_cpu_run_chain
        self._scratch = {}

    def execute(self, inputs: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        x = inputs[self.input_name]
        if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != self.k0 or not x.is_contiguous():
            raise ProviderError(f"chain kernel expects a contiguous float32 [M, {self.k0}] input, got {tuple(x.shape)} {x.dtype}")
        M = x.shape[0]
        sc = self._scratch.get(M)
        if sc is None:
            sc = (torch.empty(M * self.max_n), torch.empty(M * self.max_n))
            self._scratch[M] = sc
        out = torch.empty((M, self.n_out), dtype=torch.float32)
        self._fn(x.data_ptr(), M, self.k0, self._n, self._kinds, self._w, self._b, self._acts, self._dims,
                 out.data_ptr(), sc[0].data_ptr(), sc[1].data_ptr())
        self.stats.execution_count += 1
        return {self.output_name: out}

    def get_performance_stats(self):
        return self.stats

    @staticmethod
    def match(graph: ModelGraph):
        """The node order if the graph is such a chain, else None."""
        if len(graph.inputs) != 1 or len(graph.outputs) != 1 or not graph.nodes:
            return None
        try:
            order = graph.topological_order()
        except Exception:
            return None
        cur = graph.inputs[0].name
        seen_gemm = False
        for k, n in enumerate(order):
            if not n.inputs or n.inputs[0] != cur or len(n.outputs) != 1:
                return None
            if n.op_type == "FusedGemm" and n.attr("cpu_kernel") == "simd_gemm" and len(n.inputs) <= 3:
                w = graph.initializers.get(n.inputs[1])
                if w is None or w.dtype != torch.float32 or int(n.attr("transB", 0)):
                    return None
                if len(n.inputs) > 2 and n.inputs[2] and n.inputs[2] not in graph.initializers:
                    return None
                seen_gemm = True
            elif n.op_type == "Relu" and seen_gemm:
                pass
            elif n.op_type == "Softmax" and seen_gemm and k == len(order) - 1 and int(n.attr("axis", -1)) in (-1, 1):
                pass
            else:
                return None
            cur = n.outputs[0]
        return order if (seen_gemm and cur == graph.outputs[0].name) else None


class CpuExecutionProvider(ExecutionProvider):
    provider_id = ProviderType.CPU
    name = "CpuExecutionProvider"

    def __init__(self, thread_count: int = None, enable_simd: bool = True, numa_node: int = -1,
                 enable_fusion: bool = True, pool_name: str = "ronn-cpu"):
        cores = os.cpu_count() or 1
        self.thread_count = thread_count if thread_count else max(cores - 1, 1)
        if self.thread_count < 0:
            raise ProviderError("thread_count must be positive")
        self.enable_simd = enable_simd
        self.enable_fusion = enable_fusion
        self.numa_node = numa_node
        self.pool_name = pool_name
        self.simd_features = detect_simd_features() if enable_simd else []
        self.allocator = PooledMemoryAllocator()
        self._shutdown = False

    def get_capability(self) -> ProviderCapability:
        return ProviderCapability(
            supported_ops=set(default_registry().supported_ops()) - {"BitLinear"},
            data_types=[DataType.F32, DataType.F16, DataType.BF16, DataType.F64, DataType.I8, DataType.I32,
                        DataType.I64, DataType.U8, DataType.BOOL],
            memory_types=[MemoryType.SYSTEM],
            performance_profile=PerformanceProfile.CPU,
            resource_requirements=ResourceRequirements(cpu_features=list(self.simd_features)),
            features={"simd": list(self.simd_features), "threads": self.thread_count, "numa_node": self.numa_node})

    def configure(self, config: ProviderConfig) -> None:
        if config.thread_count is not None:
            if config.thread_count <= 0:
                raise ProviderError("thread_count must be positive")
            self.thread_count = config.thread_count
        opts = config.custom_options
        if "numa_node" in opts:
            try:
                self.numa_node = int(opts["numa_node"])
            except ValueError:
                raise ProviderError(f"invalid numa_node '{opts['numa_node']}'") from None
        if "enable_simd" in opts:
            self.enable_simd = opts["enable_simd"].lower() in ("1", "true", "yes")
            self.simd_features = detect_simd_features() if self.enable_simd else []
        if "enable_fusion" in opts:
            self.enable_fusion = opts["enable_fusion"].lower() in ("1", "true", "yes")

    def compile_graph(self, graph: ModelGraph, profiler=None) -> CompiledKernel:
        reg = default_registry()
        dev = torch.device("cpu")
        if self.enable_simd and self.enable_fusion and profiler is None:
            order = ChainKernel.match(graph)
            if order is not None:
                return ChainKernel(graph, order)

        def resolve(node, g):
            if node.attr("cpu_kernel") == "simd_gemm" and self.enable_simd:
                return _simd_gemm
            return reg.get(node.op_type).fn

        def place(name, t, users):
            return t if t.device.type == "cpu" else t.cpu()

        return build_kernel(graph, dev, resolve, place, self, profiler)

    def get_allocator(self):
        return self.allocator

    def shutdown(self) -> None:
        self._shutdown = True


def create_cpu_provider(**kw) -> CpuExecutionProvider:
    return CpuExecutionProvider(**kw)

"""GPU execution provider for B200.

The reference's GPU provider dispatches each node to a Candle library call with a host round
trip per node (crates/ronn-providers/src/gpu/provider.rs:1135-1436, 1439-1455, 1601-1613) and
its "custom kernels" are uncompiled templates (gpu/cuda_kernels.rs:317-563).  Here a graph is
compiled once: initializers are moved to the device in the session's compute dtype, GEMM weights
are stored K-major for the tcgen05 kernel, and every node resolves to a hand-written sm_100a
kernel where one exists (GEMM with fused bias/activation/residual, LayerNorm, Softmax, activations,
elementwise, embedding gather, implicit-GEMM convolution, pooling).  Remaining operators (shape
manipulation and the long tail) run as PyTorch CUDA ops on the same stream.  Tensors stay on the
device between nodes; the whole run can be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..api.errors import ProviderError
from ..core.types import (DataType, MemoryType, PerformanceProfile, ProviderCapability, ProviderConfig, ProviderType)
from ..graph.ir import ModelGraph
from ..onnx.registry import default_registry
from .base import CompiledKernel, ExecutionProvider, build_kernel

_HALF = (torch.bfloat16, torch.float16)


@dataclass
class GpuProviderConfig:
    device_ids: List[int] = field(default_factory=lambda: [0])
    primary_device_id: int = 0
    memory_limit: Optional[int] = None
    enable_mixed_precision: bool = True
    enable_tensor_cores: bool = True
    stream_count: int = 1
    enable_multi_gpu: bool = False
    enable_p2p_transfer: bool = True
    load_balancing: str = "round_robin"
    enable_custom_kernels: bool = True
    compute_dtype: Optional[str] = None     # "bf16" | "fp16" | None (keep the model's dtype)


def _dtype_of(name: Optional[str]):
    return {None: None, "bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[name]


class GpuExecutionProvider(ExecutionProvider):
    provider_id = ProviderType.GPU
    name = "GpuExecutionProvider"

    def __init__(self, config: GpuProviderConfig = None):
        if not torch.cuda.is_available():
            raise ProviderError("no CUDA device is available")
        self.config = config or GpuProviderConfig()
        self.device = torch.device("cuda", torch.cuda.current_device())
        from .. import _native
        _native.cuda()                      # fail loudly when the kernel library is missing
        self.kernel_launches = 0
        self.use_cuda_graph = False
        self._pool = None

    def set_session_options(self, opts) -> None:
        if opts.dtype:
            self.config.compute_dtype = opts.dtype
        self.use_cuda_graph = bool(getattr(opts, "use_cuda_graph", False))

    def get_allocator(self):
        """The provider's device pool (size-keyed reuse, ``memory_limit``, statistics): holds what the provider keeps
        alive across runs, e.g. the static input buffers of CUDA-graph sessions."""
        if self._pool is None:
            from .device_pool import DevicePool
            self._pool = DevicePool(self.device, self.config.memory_limit)
        return self._pool

    def shutdown(self) -> None:
        if self._pool is not None:
            self._pool.clear_pools()

    def has_tensor_cores(self) -> bool:
        return torch.cuda.get_device_capability(self.device)[0] >= 7

    def get_capability(self) -> ProviderCapability:
        return ProviderCapability(
            supported_ops=set(default_registry().supported_ops()),
            data_types=[DataType.F32, DataType.F16, DataType.BF16, DataType.I8, DataType.I32, DataType.I64,
                        DataType.U8, DataType.BOOL],
            memory_types=[MemoryType.DEVICE, MemoryType.PINNED],
            performance_profile=PerformanceProfile.GPU,
            features={"device": torch.cuda.get_device_name(self.device), "tcgen05": True,
                      "compute_capability": torch.cuda.get_device_capability(self.device)})

    def configure(self, config: ProviderConfig) -> None:
        opts = config.custom_options
        if "compute_dtype" in opts:
            self.config.compute_dtype = opts["compute_dtype"]
        if "enable_custom_kernels" in opts:
            self.config.enable_custom_kernels = opts["enable_custom_kernels"].lower() in ("1", "true", "yes")

    # ------------------------------------------------------------------ compile
    def compile_graph(self, graph: ModelGraph, profiler=None) -> CompiledKernel:
        from .gpu_ops import GpuOpTable
        cdt = _dtype_of(self.config.compute_dtype)
        table = GpuOpTable(self, graph, cdt)
        kernel = build_kernel(graph, self.device, table.resolve, table.place_const, self, profiler)
        if cdt is not None:
            kernel.input_cast = cdt
            inner = kernel.execute

            def execute(inputs, _inner=inner, _cdt=cdt):
                feed = {k: (v.to(_cdt) if v.is_floating_point() and v.dtype != _cdt else v) for k, v in inputs.items()}
                return _inner(feed)
            kernel.execute = execute
        if self.use_cuda_graph:
            kernel.execute = _GraphedExecute(kernel.execute, self.device, self.get_allocator())
        return kernel


class _GraphedExecute:
    """Replays the whole node sequence as one CUDA graph per input signature.  Inputs are copied into static
    buffers; outputs are the graph's static tensors (valid until the next run of the same session)."""

    def __init__(self, inner, device, pool=None):
        self.inner, self.device, self.graphs, self.pool = inner, device, {}, pool

    def __call__(self, inputs):
        key = tuple((k, tuple(v.shape), v.dtype) for k, v in sorted(inputs.items()))
        entry = self.graphs.get(key)
        if entry is None:
            if self.pool is not None:               # long-lived staging buffers count against the provider's limit
                static_in = {k: self.pool.tensor(v.shape, v.dtype).copy_(v) for k, v in inputs.items()}
            else:
                static_in = {k: v.clone() for k, v in inputs.items()}
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):                     # warm-up: lazy kernel attributes, workspaces, caches
                    self.inner(static_in)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                static_out = self.inner(static_in)
            entry = (g, static_in, static_out)
            self.graphs[key] = entry
        g, static_in, static_out = entry
        for k, v in inputs.items():
            static_in[k].copy_(v, non_blocking=True)
        g.replay()
        return static_out


def create_gpu_provider(**kw) -> GpuExecutionProvider:
    return GpuExecutionProvider(**kw)

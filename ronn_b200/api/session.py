"""Sessions: options, builder, inference.

API shape of the reference (crates/ronn-api/src/session.rs:14-284): ``SessionOptions`` is an
immutable builder whose ``with_*`` calls return new values (defaults O2 + CPU);
``SessionBuilder.build`` clones the graph, optimises it, obtains the requested provider (or raises
``ProviderError("Provider ... not available")``) and returns an ``InferenceSession`` whose ``run``
maps named inputs to named outputs.  Differences: execution goes through the kernel compiled by
the chosen provider in topological order (the reference interprets nodes in file order on CPU
whatever the provider, session.rs:241-274); ``num_threads`` and ``enable_profiling`` are honoured;
``run_async`` works; per-session statistics are kept.
"""
from __future__ import annotations

import asyncio
import threading
import time
from dataclasses import dataclass, replace
from typing import Dict, List, Mapping, Optional

import numpy as np
import torch

from ..core.profiling import ProfileConfig, Profiler
from ..core.types import DataType, OptimizationLevel, ProviderType
from ..graph.ir import ModelGraph
from ..graph.optimizer import OptimizationStats, Optimizer
from .errors import InferenceError, InvalidInput, ProviderError, SessionError


@dataclass(frozen=True)
class SessionOptions:
    optimization_level: OptimizationLevel = OptimizationLevel.O2
    provider_type: ProviderType = ProviderType.CPU
    num_threads: Optional[int] = None
    enable_profiling: bool = False
    dtype: Optional[str] = None            # compute dtype on the GPU provider: "fp16" | "bf16" | "fp32" | None (model's)
    tp_size: int = 1
    enable_hrm: bool = False
    use_cuda_graph: bool = False
    provider_instance: Optional[object] = None    # an ExecutionProvider object to run on (e.g. a custom-hardware provider)

    @staticmethod
    def new() -> "SessionOptions":
        return SessionOptions()

    def with_optimization_level(self, level) -> "SessionOptions":
        return replace(self, optimization_level=OptimizationLevel.parse(level))

    def with_provider(self, provider) -> "SessionOptions":
        """A provider kind ("cpu" | "gpu" | "bitnet" | "wasm" | "custom" or a ``ProviderType``), or an
        ``ExecutionProvider`` object (a custom-hardware provider, a pre-configured provider) to run on."""
        from ..providers.base import ExecutionProvider
        if isinstance(provider, ExecutionProvider):
            return replace(self, provider_type=provider.provider_id, provider_instance=provider)
        return replace(self, provider_type=ProviderType.parse(provider), provider_instance=None)

    def with_num_threads(self, n: int) -> "SessionOptions":
        return replace(self, num_threads=int(n))

    def with_profiling(self, enable: bool) -> "SessionOptions":
        return replace(self, enable_profiling=bool(enable))

    def with_dtype(self, dtype: Optional[str]) -> "SessionOptions":
        return replace(self, dtype=dtype)

    def with_tp_size(self, n: int) -> "SessionOptions":
        return replace(self, tp_size=int(n))

    def with_hrm(self, enable: bool) -> "SessionOptions":
        return replace(self, enable_hrm=bool(enable))

    def with_cuda_graph(self, enable: bool) -> "SessionOptions":
        return replace(self, use_cuda_graph=bool(enable))

    def clone(self) -> "SessionOptions":
        return replace(self)


@dataclass
class SessionStats:
    total_runs: int = 0
    total_time_ms: float = 0.0
    min_time_ms: float = 0.0
    max_time_ms: float = 0.0
    errors: int = 0

    @property
    def avg_time_ms(self) -> float:
        return self.total_time_ms / self.total_runs if self.total_runs else 0.0

    def as_dict(self) -> Dict[str, float]:
        return {"total_runs": self.total_runs, "avg_time_ms": self.avg_time_ms, "min_time_ms": self.min_time_ms,
                "max_time_ms": self.max_time_ms, "total_time_ms": self.total_time_ms, "errors": self.errors}


class SessionBuilder:
    def __init__(self, model):
        self.model = model
        self.options = SessionOptions()

    def with_options(self, options: SessionOptions) -> "SessionBuilder":
        self.options = options
        return self

    def build(self) -> "InferenceSession":
        from ..providers import create_comprehensive_provider_system, create_provider_system
        opts = self.options
        graph: ModelGraph = self.model.graph.clone()
        opt_stats = Optimizer(opts.optimization_level, opts.provider_type).optimize(graph)
        if opts.tp_size > 1:
            self._shard_for_tensor_parallel(graph, opts.tp_size)
        if opts.provider_instance is not None:
            registry = create_provider_system()
            if registry.get_provider(opts.provider_type) is not None:
                registry.unregister_provider(opts.provider_type)
            registry.register_provider(opts.provider_instance)
        elif opts.provider_type in (ProviderType.WASM, ProviderType.CUSTOM):
            registry = create_comprehensive_provider_system()
        else:
            registry = create_provider_system()
        provider = registry.get_provider(opts.provider_type)
        if provider is None:
            raise ProviderError(f"Provider {opts.provider_type.name} not available")
        if opts.num_threads and opts.provider_type == ProviderType.CPU:
            provider.thread_count = opts.num_threads
            torch.set_num_threads(max(1, min(opts.num_threads, 256)))
        if hasattr(provider, "set_session_options"):
            provider.set_session_options(opts)
        profiler = Profiler(ProfileConfig.development()) if opts.enable_profiling else None
        try:
            kernel = provider.compile_graph(graph, profiler)
        except ProviderError:
            raise
        except Exception as e:
            raise SessionError(f"failed to compile graph for {opts.provider_type.name}: {e}") from e
        sess = InferenceSession(self.model, graph, opts, registry, provider, kernel, profiler, opt_stats)
        if opts.enable_hrm:
            from ..hrm.session_router import attach_router
            attach_router(sess)
        return sess


def _shard_for_tensor_parallel(graph: ModelGraph, tp_size: int) -> None:
    """``tp_size > 1``: every rank of the default process group builds the same session and keeps its shard of the
    weights (``graph/passes/tensor_parallel.py``); the group must already exist and have ``tp_size`` ranks."""
    import torch.distributed as dist
    from ..graph.passes.tensor_parallel import TensorParallelPass
    if not (dist.is_available() and dist.is_initialized()):
        raise SessionError(f"tp_size={tp_size} needs an initialised torch.distributed process group (one process per "
                           "GPU, e.g. under torchrun)")
    if dist.get_world_size() != tp_size:
        raise SessionError(f"tp_size={tp_size} does not match the process group's world size {dist.get_world_size()}")
    from ..graph.passes.fusion import NodeFusionPass
    NodeFusionPass().run(graph)          # MatMul + Add pairs and Q / K / V projections in their fused form, at any level
    TensorParallelPass(dist.get_rank(), tp_size).run(graph)


SessionBuilder._shard_for_tensor_parallel = staticmethod(_shard_for_tensor_parallel)


def _to_tensor(v, device, name: str) -> torch.Tensor:
    if isinstance(v, torch.Tensor):
        t = v
    elif isinstance(v, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(v))
    elif isinstance(v, (list, tuple, int, float)):
        t = torch.tensor(v)
        if t.dtype == torch.float64:
            t = t.float()
    else:
        raise InvalidInput(f"input '{name}' has unsupported type {type(v).__name__}")
    if t.device != device:
        t = t.to(device, non_blocking=True)
    return t


class InferenceSession:
    def __init__(self, model, graph, options, registry, provider, kernel, profiler, opt_stats):
        self._model = model
        self._graph = graph
        self._options = options
        self._registry = registry
        self._provider = provider
        self._kernel = kernel
        self._profiler = profiler
        self._opt_stats: OptimizationStats = opt_stats
        self._stats = SessionStats()
        self._lock = threading.Lock()
        self._router = None
        self._input_names = [i.name for i in graph.inputs]

    # ------------------------------------------------------------------ accessors
    def options(self) -> SessionOptions:
        return self._options

    def graph(self) -> ModelGraph:
        return self._graph

    def provider(self):
        return self._provider

    def input_names(self) -> List[str]:
        return self._graph.input_names()

    def output_names(self) -> List[str]:
        return self._graph.output_names()

    def optimization_stats(self) -> OptimizationStats:
        return self._opt_stats

    def stats(self) -> Dict[str, float]:
        return self._stats.as_dict()

    def compilation_plan(self):
        """The kernel compiler's analysis of the optimised graph (fusion groups with cost estimates, tensor lifetimes
        and the buffer plan, planned peak bytes: ``providers/compiler.py``).  The executor uses its lifetimes to drop
        every intermediate tensor after its last reader."""
        plan = getattr(self._kernel, "plan", None)
        if plan is None:
            from ..providers.compiler import KernelCompiler
            plan = KernelCompiler.performance_preset().analyze(self._graph)
        return plan

    def profile_report(self):
        if self._profiler is None:
            raise SessionError("profiling is not enabled on this session")
        return self._profiler.report()

    # ------------------------------------------------------------------ execution
    def _validate(self, inputs: Mapping[str, object]) -> None:
        for info in self._graph.inputs:
            if info.name not in inputs:
                raise InvalidInput(f"required input '{info.name}' not provided")

    def run(self, inputs: Mapping[str, object]) -> Dict[str, torch.Tensor]:
        if not isinstance(inputs, Mapping):
            raise InvalidInput("inputs must be a mapping of input name to tensor")
        dev = self._kernel.device
        feed = {}
        for name in self._input_names:
            try:
                v = inputs[name]
            except KeyError:
                raise InvalidInput(f"required input '{name}' not provided") from None
            feed[name] = v if (type(v) is torch.Tensor and v.device == dev) else _to_tensor(v, dev, name)
        t0 = time.perf_counter()
        try:
            with torch.no_grad():
                if self._router is not None:
                    out = self._router.run(feed)
                else:
                    out = self._kernel.execute(feed)
        except Exception:
            with self._lock:
                self._stats.errors += 1
            raise
        ms = (time.perf_counter() - t0) * 1e3
        with self._lock:
            s = self._stats
            s.min_time_ms = ms if s.total_runs == 0 else min(s.min_time_ms, ms)
            s.max_time_ms = max(s.max_time_ms, ms)
            s.total_runs += 1
            s.total_time_ms += ms
        return out

    def run_numpy(self, inputs: Mapping[str, object]) -> Dict[str, np.ndarray]:
        out = self.run(inputs)
        return {k: (v.float() if v.dtype == torch.bfloat16 else v).cpu().numpy() for k, v in out.items()}

    def run_batch(self, batch: List[Mapping[str, object]]) -> List[Dict[str, torch.Tensor]]:
        return [self.run(b) for b in batch]

    async def run_async(self, inputs: Mapping[str, object]) -> Dict[str, torch.Tensor]:
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(None, self.run, inputs)

    def create_batch_processor(self, config=None):
        from .batch import BatchConfig, BatchProcessor
        return BatchProcessor(self, config or BatchConfig())

    def __repr__(self):
        return (f"InferenceSession(provider={self._options.provider_type.name}, "
                f"level={self._options.optimization_level.name}, nodes={len(self._graph.nodes)})")

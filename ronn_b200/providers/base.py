"""Execution-provider contracts (crates/ronn-core/src/types.rs:153-165 CompiledKernel,
:192-213 ExecutionProvider, :294-303 TensorAllocator).

A provider compiles a (sub)graph into a ``CompiledKernel``: a pre-resolved, topologically
ordered list of callables over a slot table.  Unlike the reference, where the provider chosen
on the session is looked up but never used (crates/ronn-api/src/session.rs:105-131), the
session executes through the kernel its provider compiled.
"""
from __future__ import annotations

import time
from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from ..api.errors import InferenceError, ProviderError, UnsupportedOperator
from ..core.types import (KernelStats, MemoryInfo, MemoryUsage, OperatorSpec, ProviderCapability, ProviderConfig,
                          ProviderType, TensorBuffer)
from ..graph.ir import ModelGraph, SubGraph


class TensorAllocator(ABC):
    @abstractmethod
    def allocate(self, shape: Sequence[int], dtype) -> TensorBuffer: ...

    @abstractmethod
    def deallocate(self, buf: TensorBuffer) -> None: ...

    @abstractmethod
    def get_memory_info(self) -> MemoryInfo: ...


class ExecContext:
    """Per-node context handed to operator functions."""
    __slots__ = ("num_outputs", "device", "provider")

    def __init__(self, num_outputs=1, device=None, provider=None):
        self.num_outputs = num_outputs
        self.device = device
        self.provider = provider


class Step:
    __slots__ = ("fn", "in_slots", "out_slots", "attrs", "ctx", "name", "op_type")

    def __init__(self, fn, in_slots, out_slots, attrs, ctx, name, op_type):
        self.fn, self.in_slots, self.out_slots = fn, in_slots, out_slots
        self.attrs, self.ctx, self.name, self.op_type = attrs, ctx, name, op_type


class CompiledKernel:
    """Slot-table interpreter: constants are bound once, inputs are written per run."""

    def __init__(self, steps: List[Step], n_slots: int, const_slots: Dict[int, torch.Tensor],
                 input_slots: Dict[str, int], output_slots: Dict[str, int], device: torch.device,
                 profiler=None, release_after: Optional[List[List[int]]] = None, plan=None):
        self.steps = steps
        self.n_slots = n_slots
        self.const_slots = const_slots
        self.input_slots = input_slots
        self.output_slots = output_slots
        self.device = device
        self.stats = KernelStats()
        self.profiler = profiler
        # slots whose last reader is step k (from the compiler's lifetime analysis): dropped right after it, so an
        # intermediate tensor lives only as long as the graph needs it instead of until the end of the run
        self.release_after = release_after
        self.plan = plan
        self._template: List[Any] = [None] * n_slots
        for k, v in const_slots.items():
            self._template[k] = v

    def execute(self, inputs: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        t0 = time.perf_counter()
        slots = list(self._template)
        for name, slot in self.input_slots.items():
            slots[slot] = inputs[name]
        prof = self.profiler
        release = self.release_after
        for k, st in enumerate(self.steps):
            args = [slots[s] if s >= 0 else None for s in st.in_slots]
            try:
                if prof is not None and prof.enabled:
                    with prof.scope(st.name, st.op_type, device=self.device):
                        outs = st.fn(args, st.attrs, st.ctx)
                else:
                    outs = st.fn(args, st.attrs, st.ctx)
            except (InferenceError, UnsupportedOperator):
                raise
            except Exception as e:
                raise InferenceError(f"node '{st.name}' ({st.op_type}) failed: {e}") from e
            for s, o in zip(st.out_slots, outs):
                if s >= 0:
                    slots[s] = o
            if release is not None:
                args = None
                for s in release[k]:
                    slots[s] = None
        out = {name: slots[s] for name, s in self.output_slots.items()}
        self.stats.record((time.perf_counter() - t0) * 1e6)
        return out

    def get_memory_usage(self) -> MemoryUsage:
        n = sum(t.numel() * t.element_size() for t in self.const_slots.values() if isinstance(t, torch.Tensor))
        return MemoryUsage(peak_bytes=n, current_bytes=n, allocation_count=len(self.const_slots))

    def get_performance_stats(self) -> KernelStats:
        return self.stats


class ExecutionProvider(ABC):
    provider_id: ProviderType = ProviderType.CPU
    name = "provider"

    @abstractmethod
    def get_capability(self) -> ProviderCapability: ...

    def can_handle(self, ops: Sequence[OperatorSpec]) -> List[bool]:
        sup = self.get_capability().supported_ops
        return [o.op_type in sup for o in ops]

    @abstractmethod
    def compile_graph(self, graph: ModelGraph, profiler=None) -> CompiledKernel: ...

    def compile_subgraph(self, subgraph: SubGraph, initializers: Optional[Dict[str, torch.Tensor]] = None):
        from ..graph.ir import TensorInfo
        from ..core.types import DataType
        if not subgraph.nodes:
            raise ProviderError("cannot compile an empty subgraph")
        g = ModelGraph.from_nodes([n.clone() for n in subgraph.nodes])
        g.initializers = dict(initializers or {})
        g.inputs = [TensorInfo(i, [], DataType.F32) for i in subgraph.inputs if i not in g.initializers]
        g.outputs = [TensorInfo(o, [], DataType.F32) for o in subgraph.outputs]
        unsupported = [n.op_type for n in g.nodes if n.op_type not in self.get_capability().supported_ops]
        if unsupported:
            raise ProviderError(f"{self.name} does not support operators: {sorted(set(unsupported))}")
        return self.compile_graph(g)

    def get_allocator(self) -> Optional[TensorAllocator]:
        return None

    def configure(self, config: ProviderConfig) -> None:
        pass

    def shutdown(self) -> None:
        pass


def build_kernel(graph: ModelGraph, device: torch.device, resolve: Callable, place_const: Callable,
                 provider=None, profiler=None) -> CompiledKernel:
    """Common compile routine: topological order, slot assignment, constant placement.

    ``resolve(node, graph) -> fn`` picks the callable of a node; ``place_const(name, tensor, users) -> tensor``
    moves an initializer to where the provider wants it."""
    order = graph.topological_order()
    slot_of: Dict[str, int] = {}

    def slot(name: str) -> int:
        if not name:
            return -1
        if name not in slot_of:
            slot_of[name] = len(slot_of)
        return slot_of[name]

    cons = graph.consumers()
    consts = {}
    for name, t in graph.initializers.items():
        if name in cons or name in graph.output_names():
            consts[slot(name)] = place_const(name, t, cons.get(name, []))
    input_slots = {i.name: slot(i.name) for i in graph.inputs}
    steps = []
    for n in order:
        fn = resolve(n, graph)
        ins = [slot(i) for i in n.inputs]
        outs = [slot(o) for o in n.outputs]
        ctx = ExecContext(len(n.outputs), device, provider)
        steps.append(Step(fn, ins, outs, n.attributes, ctx, n.name or f"node_{n.id}", n.op_type))
    output_slots = {}
    for o in graph.outputs:
        if o.name not in slot_of:
            raise ProviderError(f"graph output '{o.name}' is never produced")
        output_slots[o.name] = slot_of[o.name]
    # lifetimes from the kernel compiler's memory plan (crates/ronn-providers/src/compiler.rs:430-520 plans buffers but
    # nothing there consumes the plan): a produced tensor is released after its last reader
    from .compiler import KernelCompiler
    plan = KernelCompiler.performance_preset().analyze(graph)
    keep = set(output_slots.values()) | set(consts) | set(input_slots.values())
    release_after: List[List[int]] = [[] for _ in steps]
    for b in plan.memory_plan:
        s = slot_of.get(b.tensor)
        if s is not None and s not in keep and 0 <= b.last_use < len(steps):
            release_after[b.last_use].append(s)
    return CompiledKernel(steps, len(slot_of), consts, input_slots, output_slots, device, profiler,
                          release_after=release_after, plan=plan)

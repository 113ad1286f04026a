"""Sub-graph analysis: fusion groups, cost estimate, memory plan
(crates/ronn-providers/src/compiler.rs:14-631).

Topological order, greedy linear fusion-group growth up to ``max_fusion_depth`` over the reference's
``can_fuse`` table (Add/Mul/Sub->Relu, Add->Add, Mul->Mul, Conv->BatchNormalization,
BatchNormalization->Relu, MatMul/Gemm->Add), group classification {None, ElementWise, ConvBnRelu,
MatMulBias, Custom}, multiplicative cost factors (0.7 / 0.6 / 0.8 / 0.9) and a lifetime-based
memory plan with same-size buffer reuse.  Shapes come from the graph's value_info when present
(the reference guesses [32,32] f32 for everything).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..graph.ir import ModelGraph, SubGraph


class FusionType(enum.Enum):
    NONE = "none"
    ELEMENTWISE = "elementwise"
    CONV_BN_RELU = "conv_bn_relu"
    MATMUL_BIAS = "matmul_bias"
    CUSTOM = "custom"


_CAN_FUSE = {("Add", "Relu"), ("Mul", "Relu"), ("Sub", "Relu"), ("Add", "Add"), ("Mul", "Mul"),
             ("Conv", "BatchNormalization"), ("BatchNormalization", "Relu"), ("MatMul", "Add"), ("Gemm", "Add"),
             ("Conv", "Relu")}
_COST = {FusionType.NONE: 1.0, FusionType.ELEMENTWISE: 0.7, FusionType.CONV_BN_RELU: 0.6, FusionType.MATMUL_BIAS: 0.8,
         FusionType.CUSTOM: 0.9}
_OP_COST = {"Conv": 100.0, "MatMul": 50.0, "Gemm": 50.0, "BatchNormalization": 5.0, "Softmax": 8.0,
            "LayerNormalization": 8.0, "Attention": 80.0}


@dataclass
class FusionConfig:
    max_fusion_depth: int = 6
    enable_conv_fusion: bool = True
    enable_elementwise_fusion: bool = True


@dataclass
class MemoryConfig:
    max_memory_overhead: float = 0.3
    enable_reuse: bool = True


@dataclass
class FusionGroup:
    node_ids: List[int]
    op_types: List[str]
    fusion_type: FusionType
    estimated_cost: float


@dataclass
class BufferAssignment:
    tensor: str
    buffer: int
    size_bytes: int
    first_use: int
    last_use: int


@dataclass
class CompilationPlan:
    order: List[int]
    groups: List[FusionGroup]
    memory_plan: List[BufferAssignment]
    total_cost: float
    peak_bytes: int
    buffers: int


class KernelCompiler:
    def __init__(self, fusion: FusionConfig = None, memory: MemoryConfig = None):
        self.fusion = fusion or FusionConfig()
        self.memory = memory or MemoryConfig()

    @staticmethod
    def performance_preset() -> "KernelCompiler":
        return KernelCompiler(FusionConfig(6, True, True), MemoryConfig(0.3, True))

    @staticmethod
    def memory_preset() -> "KernelCompiler":
        return KernelCompiler(FusionConfig(3, False, True), MemoryConfig(0.1, True))

    def can_fuse(self, a: str, b: str) -> bool:
        if not self.fusion.enable_conv_fusion and "Conv" in (a, b):
            return False
        if not self.fusion.enable_elementwise_fusion and (a, b) in {("Add", "Relu"), ("Mul", "Relu"), ("Sub", "Relu"),
                                                                   ("Add", "Add"), ("Mul", "Mul")}:
            return False
        return (a, b) in _CAN_FUSE

    @staticmethod
    def classify(ops: List[str]) -> FusionType:
        if len(ops) < 2:
            return FusionType.NONE
        if ops[0] == "Conv":
            return FusionType.CONV_BN_RELU
        if ops[0] in ("MatMul", "Gemm") and ops[1] == "Add":
            return FusionType.MATMUL_BIAS
        if all(o in ("Add", "Mul", "Sub", "Relu", "Sigmoid", "Tanh") for o in ops):
            return FusionType.ELEMENTWISE
        return FusionType.CUSTOM

    def analyze(self, graph: ModelGraph) -> CompilationPlan:
        order = graph.topological_order()
        cons = graph.consumers()
        outputs = set(graph.output_names())
        placed = set()
        groups: List[FusionGroup] = []
        for n in order:
            if n.id in placed:
                continue
            chain = [n]
            cur = n
            while len(chain) < self.fusion.max_fusion_depth:
                out = cur.outputs[0] if cur.outputs else None
                users = cons.get(out, []) if out else []
                if out in outputs or len(users) != 1:
                    break
                nxt = users[0]
                if nxt.id in placed or not self.can_fuse(cur.op_type, nxt.op_type):
                    break
                chain.append(nxt)
                cur = nxt
            for c in chain:
                placed.add(c.id)
            ops = [c.op_type for c in chain]
            ft = self.classify(ops)
            base = sum(_OP_COST.get(o, 1.0) for o in ops)
            groups.append(FusionGroup([c.id for c in chain], ops, ft, base * _COST[ft]))
        mem, peak, nbuf = self._memory_plan(graph, order)
        return CompilationPlan([n.id for n in order], groups, mem, sum(g.estimated_cost for g in groups), peak, nbuf)

    def analyze_subgraph(self, sg: SubGraph) -> CompilationPlan:
        g = ModelGraph.from_nodes([n.clone() for n in sg.nodes])
        return self.analyze(g)

    def _size_of(self, graph: ModelGraph, name: str) -> int:
        info = graph.value_info.get(name)
        if info is not None and info.shape and all(d > 0 for d in info.shape):
            n = 1
            for d in info.shape:
                n *= d
            return n * info.data_type.itemsize
        return 32 * 32 * 4

    def _memory_plan(self, graph: ModelGraph, order) -> Tuple[List[BufferAssignment], int, int]:
        pos = {n.id: k for k, n in enumerate(order)}
        first: Dict[str, int] = {}
        last: Dict[str, int] = {}
        for n in order:
            for o in n.outputs:
                if o:
                    first[o] = pos[n.id]
                    last.setdefault(o, pos[n.id])
            for i in n.inputs:
                if i in first:
                    last[i] = pos[n.id]
        for o in graph.output_names():
            if o in first:
                last[o] = len(order)
        free: Dict[int, List[int]] = {}
        assigns: List[BufferAssignment] = []
        live: List[Tuple[int, int, int]] = []     # (last_use, buffer, size)
        nbuf, cur, peak = 0, 0, 0
        for name in sorted(first, key=lambda t: first[t]):
            t = first[name]
            for item in [x for x in live if x[0] < t]:
                live.remove(item)
                cur -= item[2]
                if self.memory.enable_reuse:
                    free.setdefault(item[2], []).append(item[1])
            size = self._size_of(graph, name)
            if self.memory.enable_reuse and free.get(size):
                buf = free[size].pop()
            else:
                buf = nbuf
                nbuf += 1
            cur += size
            peak = max(peak, cur)
            live.append((last[name], buf, size))
            assigns.append(BufferAssignment(name, buf, size, t, last[name]))
        return assigns, peak, nbuf

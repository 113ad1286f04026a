"""Graph IR.

Same vocabulary as the reference (crates/ronn-core/src/types.rs:107-156 ModelGraph /
GraphNode / GraphEdge, :349-358 SubGraph; crates/ronn-core/src/graph.rs:29-47 add/get,
:117-151 validate, :222-260 topological_sort, :263-335 extract_subgraph, :347-389
statistics, :424-513 GraphBuilder), with one behavioural difference: edges are real.
The reference's loader builds graphs with ``from_nodes`` and no edges (graph.rs:75-83),
which is why its passes cannot find successors; here producer->consumer edges are derived
from tensor names, and the algorithms run in the native library on interned ids.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..api.errors import GraphError
from ..core.types import DataType


@dataclass
class TensorInfo:
    name: str
    shape: List[int]                       # dynamic dims are 0 (as in the reference loader)
    data_type: DataType
    dim_params: List[Optional[str]] = field(default_factory=list)   # symbolic names of dynamic dims

    def __post_init__(self):
        if not self.dim_params:
            self.dim_params = [None] * len(self.shape)


@dataclass
class GraphNode:
    id: int
    op_type: str
    inputs: List[str]
    outputs: List[str]
    attributes: Dict[str, Any] = field(default_factory=dict)
    name: Optional[str] = None
    domain: str = ""

    def attr(self, key: str, default=None):
        return self.attributes.get(key, default)

    def clone(self) -> "GraphNode":
        return GraphNode(self.id, self.op_type, list(self.inputs), list(self.outputs), dict(self.attributes),
                         self.name, self.domain)


@dataclass
class GraphEdge:
    from_node: int
    to_node: int
    tensor_name: str


@dataclass
class SubGraph:
    nodes: List[GraphNode]
    edges: List[GraphEdge]
    inputs: List[str]
    outputs: List[str]


@dataclass
class GraphStatistics:
    node_count: int
    edge_count: int
    input_count: int
    output_count: int
    op_type_counts: Dict[str, int]
    max_depth: int


class ModelGraph:
    """A dataflow graph over named tensors, with weights held as initializers."""

    def __init__(self):
        self.nodes: List[GraphNode] = []
        self.inputs: List[TensorInfo] = []
        self.outputs: List[TensorInfo] = []
        self.initializers: Dict[str, torch.Tensor] = {}
        self.metadata: Dict[str, str] = {}
        self.value_info: Dict[str, TensorInfo] = {}
        self.name: str = ""
        self._next_id = 0

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_nodes(nodes: Iterable[GraphNode]) -> "ModelGraph":
        g = ModelGraph()
        for n in nodes:
            g.nodes.append(n)
            g._next_id = max(g._next_id, n.id + 1)
        return g

    def add_node(self, op_type: str, inputs: Sequence[str], outputs: Sequence[str],
                 attributes: Optional[Dict[str, Any]] = None, name: Optional[str] = None,
                 domain: str = "", index: Optional[int] = None) -> GraphNode:
        node = GraphNode(self._next_id, op_type, list(inputs), list(outputs), dict(attributes or {}), name, domain)
        self._next_id += 1
        if index is None:
            self.nodes.append(node)
        else:
            self.nodes.insert(index, node)
        return node

    def remove_nodes(self, ids: Iterable[int]) -> int:
        ids = set(ids)
        before = len(self.nodes)
        self.nodes = [n for n in self.nodes if n.id not in ids]
        return before - len(self.nodes)

    def get_node(self, node_id: int) -> Optional[GraphNode]:
        for n in self.nodes:
            if n.id == node_id:
                return n
        return None

    def node_count(self) -> int:
        return len(self.nodes)

    def input_names(self) -> List[str]:
        return [i.name for i in self.inputs]

    def output_names(self) -> List[str]:
        return [o.name for o in self.outputs]

    def clone(self) -> "ModelGraph":
        g = ModelGraph()
        g.nodes = [n.clone() for n in self.nodes]
        g.inputs = list(self.inputs)
        g.outputs = list(self.outputs)
        g.initializers = dict(self.initializers)      # tensors are shared, not copied
        g.metadata = dict(self.metadata)
        g.value_info = dict(self.value_info)
        g.name = self.name
        g._next_id = self._next_id
        return g

    # ------------------------------------------------------------------ derived structure
    def producers(self) -> Dict[str, GraphNode]:
        out = {}
        for n in self.nodes:
            for o in n.outputs:
                if o:
                    out[o] = n
        return out

    def consumers(self) -> Dict[str, List[GraphNode]]:
        out: Dict[str, List[GraphNode]] = {}
        for n in self.nodes:
            for i in n.inputs:
                if i:
                    out.setdefault(i, []).append(n)
        return out

    @property
    def edges(self) -> List[GraphEdge]:
        prod = self.producers()
        es = []
        for n in self.nodes:
            for i in n.inputs:
                p = prod.get(i)
                if p is not None:
                    es.append(GraphEdge(p.id, n.id, i))
        return es

    def fresh_name(self, base: str) -> str:
        used = set(self.initializers) | {o for n in self.nodes for o in n.outputs} | set(self.input_names())
        if base not in used:
            return base
        k = 1
        while f"{base}_{k}" in used:
            k += 1
        return f"{base}_{k}"

    # ------------------------------------------------------------------ native algorithms
    def _native_graph(self) -> Tuple[Any, Dict[str, int]]:
        lib = _native.host()
        intern: Dict[str, int] = {}

        def vid(name: str) -> int:
            if name not in intern:
                intern[name] = len(intern)
            return intern[name]

        h = lib.ronn_graph_new()
        for n in self.nodes:
            ins = np.asarray([vid(i) for i in n.inputs if i], dtype=np.int32)
            outs = np.asarray([vid(o) for o in n.outputs if o], dtype=np.int32)
            lib.ronn_graph_add_node(h, ins.ctypes.data_as(_native.c_i32p), len(ins),
                                    outs.ctypes.data_as(_native.c_i32p), len(outs))
        return h, intern

    def topological_order(self) -> List[GraphNode]:
        """Kahn order, stable with respect to the current node order.  Raises on cycles."""
        if not self.nodes:
            return []
        lib = _native.host()
        h, _ = self._native_graph()
        try:
            order = np.empty(len(self.nodes), dtype=np.int32)
            placed = lib.ronn_graph_toposort(h, order.ctypes.data_as(_native.c_i32p))
        finally:
            lib.ronn_graph_free(h)
        if placed != len(self.nodes):
            raise GraphError("graph contains a cycle")
        return [self.nodes[i] for i in order]

    def topological_sort(self) -> List[int]:
        return [n.id for n in self.topological_order()]

    def sort_in_place(self) -> None:
        self.nodes = self.topological_order()

    def validate(self) -> None:
        """Duplicate ids, duplicate producers, cycles, undefined node inputs, unproduced outputs."""
        ids = set()
        for n in self.nodes:
            if n.id in ids:
                raise GraphError(f"duplicate node id {n.id}")
            ids.add(n.id)
            if not n.op_type:
                raise GraphError(f"node {n.name or n.id} has an empty op_type")
        names = [i.name for i in self.inputs]
        if len(set(names)) != len(names):
            raise GraphError("duplicate graph input name")
        if not self.nodes:
            known = set(names) | set(self.initializers)
            for o in self.outputs:
                if o.name not in known:
                    raise GraphError(f"graph output '{o.name}' is never produced")
            return
        lib = _native.host()
        h, intern = self._native_graph()
        rev = {v: k for k, v in intern.items()}
        try:
            def ids_of(xs):
                arr = []
                for x in xs:
                    if x not in intern:
                        intern[x] = len(intern)
                        rev[intern[x]] = x
                    arr.append(intern[x])
                return np.asarray(arr, dtype=np.int32)
            sources = ids_of(list(names) + list(self.initializers.keys()))
            outputs = ids_of([o.name for o in self.outputs])
            detail = C.c_int32(-1)
            rc = lib.ronn_graph_validate(h, sources.ctypes.data_as(_native.c_i32p), len(sources),
                                         outputs.ctypes.data_as(_native.c_i32p), len(outputs), C.byref(detail))
        finally:
            lib.ronn_graph_free(h)
        if rc == 1:
            raise GraphError(f"tensor '{rev.get(detail.value)}' is produced by more than one node")
        if rc == 2:
            n = self.nodes[detail.value]
            raise GraphError(f"graph contains a cycle (through node '{n.name or n.id}')")
        if rc == 3:
            raise GraphError(f"graph output '{rev.get(detail.value)}' is never produced")
        if rc == 4:
            raise GraphError(f"tensor '{rev.get(detail.value)}' is consumed but never produced or provided")

    def live_node_ids(self, outputs: Optional[Sequence[str]] = None) -> set:
        """Ids of the nodes that contribute to the given outputs (default: the graph outputs)."""
        if not self.nodes:
            return set()
        lib = _native.host()
        h, intern = self._native_graph()
        try:
            outs = np.asarray([intern[o] for o in (outputs or self.output_names()) if o in intern], dtype=np.int32)
            live = np.zeros(len(self.nodes), dtype=np.uint8)
            lib.ronn_graph_live(h, outs.ctypes.data_as(_native.c_i32p), len(outs),
                                live.ctypes.data_as(_native.c_u8p))
        finally:
            lib.ronn_graph_free(h)
        return {self.nodes[i].id for i in np.nonzero(live)[0]}

    def depth(self) -> int:
        if not self.nodes:
            return 0
        lib = _native.host()
        h, _ = self._native_graph()
        try:
            return int(lib.ronn_graph_depth(h))
        finally:
            lib.ronn_graph_free(h)

    def statistics(self) -> GraphStatistics:
        counts: Dict[str, int] = {}
        for n in self.nodes:
            counts[n.op_type] = counts.get(n.op_type, 0) + 1
        return GraphStatistics(len(self.nodes), len(self.edges), len(self.inputs), len(self.outputs), counts,
                               max(self.depth(), 0))

    def extract_subgraph(self, node_ids: Sequence[int]) -> SubGraph:
        idset = set(node_ids)
        nodes = [n.clone() for n in self.nodes if n.id in idset]
        if len(nodes) != len(idset):
            raise GraphError("extract_subgraph: unknown node id")
        produced = {o for n in nodes for o in n.outputs if o}
        consumed_inside = {i for n in nodes for i in n.inputs if i}
        inputs = [i for i in dict.fromkeys(i for n in nodes for i in n.inputs if i) if i not in produced]
        cons = self.consumers()
        graph_outs = set(self.output_names())
        outputs = []
        for n in nodes:
            for o in n.outputs:
                if not o:
                    continue
                ext = any(c.id not in idset for c in cons.get(o, []))
                if ext or o in graph_outs or o not in consumed_inside:
                    outputs.append(o)
        edges = [e for e in self.edges if e.from_node in idset and e.to_node in idset]
        return SubGraph(nodes, edges, inputs, outputs)


class GraphBuilder:
    """Fluent construction helper (crates/ronn-core/src/graph.rs:424-513)."""

    def __init__(self):
        self.graph = ModelGraph()

    def add_input(self, name: str, shape: Sequence[int] = (), dtype: DataType = DataType.F32) -> "GraphBuilder":
        self.graph.inputs.append(TensorInfo(name, list(shape), dtype))
        return self

    def add_output(self, name: str, shape: Sequence[int] = (), dtype: DataType = DataType.F32) -> "GraphBuilder":
        self.graph.outputs.append(TensorInfo(name, list(shape), dtype))
        return self

    def add_initializer(self, name: str, tensor: torch.Tensor) -> "GraphBuilder":
        self.graph.initializers[name] = tensor
        return self

    def add_op(self, op_type: str, inputs: Sequence[str], outputs: Sequence[str], name: Optional[str] = None,
               domain: str = "", **attributes) -> "GraphBuilder":
        self.graph.add_node(op_type, inputs, outputs, attributes, name, domain)
        return self

    def build(self, validate: bool = True) -> ModelGraph:
        if validate:
            self.graph.validate()
        return self.graph

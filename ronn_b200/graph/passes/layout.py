"""Layout optimisation: run convolution chains in NHWC.

The reference pass counts conv-like ops to choose between NCHW and NHWC and then inserts
no transform at all (crates/ronn-graph/src/passes/layout.rs:15-73).  This pass does the
rewrite: when the graph's image-shaped tensors flow only through layout-aware operators
(Conv/FusedConv, pooling, BatchNormalization, elementwise Add/Relu, GlobalAveragePool),
those nodes get ``data_format="NHWC"``, convolution weights are permuted once to
[Cout, R, S, Cin], and a single Transpose is inserted on each NCHW graph input that feeds
the region.  Exits need no Transpose when they go through GlobalAveragePool -> Flatten
(an [N,1,1,C] tensor flattens to the same [N,C]); any other exit gets a Transpose back.
NHWC is what the sm_100a implicit-GEMM convolution consumes (channels innermost = K-major
operand rows for the tensor core).
"""
from __future__ import annotations

from typing import Dict, Set

from ..ir import ModelGraph
from .base import OptimizationPass, PassStats

_CONV = {"Conv", "FusedConv"}
_SPATIAL = {"MaxPool", "AveragePool", "GlobalAveragePool", "BatchNormalization"}
_ELEMENTWISE = {"Relu", "Add", "Sigmoid", "Tanh", "LeakyRelu", "Identity", "Mul", "Sub", "Clip"}


def choose_layout(graph: ModelGraph) -> str:
    """The reference's vote: conv-like ops outnumbering half of the rest -> keep image layout work worthwhile."""
    conv_like = sum(1 for n in graph.nodes if n.op_type in _CONV | _SPATIAL)
    other = len(graph.nodes) - conv_like
    return "NHWC" if conv_like > other / 2 and conv_like > 0 else "NCHW"


class LayoutOptimizationPass(OptimizationPass):
    name = "LayoutOptimization"

    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        if graph.metadata.get("ronn.layout") == "NHWC" or choose_layout(graph) != "NHWC":
            return stats
        if any(n.attr("data_format") == "NHWC" for n in graph.nodes):
            return stats
        # --- region: tensors known to be 4-D images
        image: Set[str] = set()
        region = []
        for n in graph.topological_order():
            if n.op_type in _CONV:
                w = graph.initializers.get(n.inputs[1])
                if w is None or w.dim() != 4:
                    return stats
                region.append(n)
                image.add(n.inputs[0])
                image.update(o for o in n.outputs if o)
                if len(n.inputs) > 3 and n.inputs[3]:
                    image.add(n.inputs[3])
            elif n.op_type in _SPATIAL and n.inputs[0] in image:
                region.append(n)
                image.update(o for o in n.outputs if o)
            elif n.op_type in _ELEMENTWISE and any(i in image for i in n.inputs):
                # every tensor operand must be an image of the region (constants would need broadcasting care)
                if not all((i in image) for i in n.inputs if i):
                    return stats
                region.append(n)
                image.update(o for o in n.outputs if o)
        if not region:
            return stats
        region_ids = {n.id for n in region}
        cons = graph.consumers()
        gap_outs = {n.outputs[0] for n in region if n.op_type == "GlobalAveragePool"}
        produced = {o for n in region for o in n.outputs if o}
        outputs = set(graph.output_names())
        # --- exits: tensors PRODUCED inside the region that someone outside reads in NCHW.  Entry tensors are not
        # exits: their other consumers keep reading the original NCHW tensor.
        exits: Dict[str, list] = {}
        for t in sorted(produced):
            outside = [c for c in cons.get(t, []) if c.id not in region_ids
                       and not (t in gap_outs and c.op_type in ("Flatten", "Reshape", "Squeeze"))]
            if outside or (t in outputs and t not in gap_outs):
                exits[t] = outside
        # --- entries: image tensors not produced inside the region
        entries = sorted(t for t in image if t not in produced)
        if any(t in graph.initializers for t in entries):
            return stats
        # --- rewrite
        for n in region:
            n.attributes["data_format"] = "NHWC"
            if n.op_type in _CONV:
                wname = n.inputs[1]
                new = graph.fresh_name(wname + "_nhwc")
                graph.initializers[new] = graph.initializers[wname].permute(0, 2, 3, 1).contiguous()
                n.inputs[1] = new
            stats.nodes_modified += 1
        for t in entries:
            new = graph.fresh_name(t + "_nhwc")
            first = min((k for k, n in enumerate(graph.nodes) if t in n.inputs and n.id in region_ids))
            for n in region:
                n.inputs = [new if i == t else i for i in n.inputs]
            graph.add_node("Transpose", [t], [new], {"perm": [0, 2, 3, 1]}, name=graph.fresh_name(f"to_nhwc_{t}"), index=first)
        for t, outside in exits.items():
            idx = max(k for k, n in enumerate(graph.nodes) if t in n.outputs) + 1
            if t in outputs:
                # graph output: the public name stays on the NCHW tensor; the region works on a renamed NHWC tensor and
                # outside consumers (which already read `t`) need no change
                inner = graph.fresh_name(t + "__nhwc")
                for n in region:
                    n.outputs = [inner if o == t else o for o in n.outputs]
                    n.inputs = [inner if i == t else i for i in n.inputs]
                graph.add_node("Transpose", [inner], [t], {"perm": [0, 3, 1, 2]}, name=graph.fresh_name(f"to_nchw_{t}"), index=idx)
            else:
                new = graph.fresh_name(t + "_nchw")
                graph.add_node("Transpose", [t], [new], {"perm": [0, 3, 1, 2]}, name=graph.fresh_name(f"to_nchw_{t}"), index=idx)
                for c in outside:
                    c.inputs = [new if i == t else i for i in c.inputs]
        graph.metadata["ronn.layout"] = "NHWC"
        graph.sort_in_place()
        return stats

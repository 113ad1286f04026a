"""Constant folding.

The reference pass can never fire: it has no access to initializers and its
``all_inputs_constant`` always answers false (crates/ronn-graph/src/passes/constant_folding.rs:15-57).
This one evaluates every node whose inputs are all initializers (or outputs of ``Constant``
nodes) through the operator registry on the CPU and replaces it by an initializer.
"""
from __future__ import annotations

import torch

from ...onnx.registry import default_registry
from ..ir import ModelGraph
from .base import OptimizationPass, PassStats

# ops with no tensor inputs or whose value depends on runtime shapes/state are left alone
_NEVER = {"RandomNormal", "RandomUniform", "RandomNormalLike", "RandomUniformLike", "Dropout", "BitLinear"}
_MAX_ELEMS = 1 << 26


class ConstantFoldingPass(OptimizationPass):
    name = "ConstantFolding"

    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        reg = default_registry()
        outputs = set(graph.output_names())
        changed = True
        while changed:
            changed = False
            for node in list(graph.nodes):
                if node.op_type in _NEVER or not reg.has(node.op_type):
                    continue
                if node.op_type != "Constant" and not node.inputs:
                    continue
                if any(i and i not in graph.initializers for i in node.inputs):
                    continue
                if any(o in outputs for o in node.outputs) and node.op_type == "Constant" and False:
                    continue
                ins = [graph.initializers[i] if i else None for i in node.inputs]
                try:
                    with torch.no_grad():
                        outs = reg.get(node.op_type).execute(ins, node.attributes, None)
                except Exception:
                    continue          # leave the node for the runtime to report
                if any(o.numel() > _MAX_ELEMS for o in outs):
                    continue
                for name, val in zip(node.outputs, outs):
                    if name:
                        graph.initializers[name] = val.contiguous() if isinstance(val, torch.Tensor) else val
                graph.remove_nodes([node.id])
                stats.nodes_removed += 1
                changed = True
        return stats

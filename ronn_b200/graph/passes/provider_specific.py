"""Provider-specific passes.

``CpuOptimizationPass`` and ``GpuOptimizationPass`` return 0 in the reference
(crates/ronn-graph/src/passes/provider_specific.rs:7-87).  Here:

* CPU: weights of FusedGemm/MatMul/Gemm nodes are made contiguous fp32 row-major once and the
  node is tagged for the native SIMD GEMM when it is small enough for the call to beat a
  framework dispatch (batch-1 MLP case).
* GPU: chains of elementwise nodes are collapsed into one com.ronn::FusedElementwise node so a
  chain costs one launch ("aggressive elementwise fusion to cut launches").
"""
from __future__ import annotations

import torch

from ..ir import ModelGraph
from .base import OptimizationPass, PassStats

RONN = "com.ronn"
_UNARY = {"Relu", "Sigmoid", "Tanh", "Gelu", "Neg", "Abs", "Exp", "Sqrt", "Swish"}
_BINARY = {"Add", "Mul", "Sub", "Div"}


class CpuOptimizationPass(OptimizationPass):
    name = "CpuOptimization"

    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        for n in graph.nodes:
            if n.op_type not in ("FusedGemm", "MatMul", "Gemm") or n.attr("cpu_kernel"):
                continue
            w = graph.initializers.get(n.inputs[1]) if len(n.inputs) > 1 else None
            if w is None or w.dim() != 2 or w.dtype != torch.float32:
                continue
            if n.op_type == "Gemm" and (int(n.attr("transA", 0)) or float(n.attr("alpha", 1.0)) != 1.0
                                        or float(n.attr("beta", 1.0)) != 1.0):
                continue
            if n.attr("activation", "") not in ("", "Relu") or len(n.inputs) > 3:
                continue
            if int(n.attr("transB", 0)):
                new = graph.fresh_name(n.inputs[1] + "_kn")
                graph.initializers[new] = w.t().contiguous()
                n.inputs[1] = new
                n.attributes["transB"] = 0
            elif not w.is_contiguous():
                graph.initializers[n.inputs[1]] = w.contiguous()
            n.attributes["cpu_kernel"] = "simd_gemm"
            stats.nodes_modified += 1
        return stats


class GpuOptimizationPass(OptimizationPass):
    name = "GpuOptimization"

    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        outputs = set(graph.output_names())
        progress = True
        while progress:
            progress = False
            cons = graph.consumers()
            for head in graph.nodes:
                if not self._elementwise(head, graph) or head.op_type == "FusedElementwise":
                    continue
                chain = [head]
                cur = head
                while True:
                    out = cur.outputs[0]
                    users = cons.get(out, [])
                    if out in outputs or len(users) != 1:
                        break
                    nxt = users[0]
                    if not self._elementwise(nxt, graph) or nxt.inputs[0] != out or nxt.op_type == "FusedElementwise":
                        break
                    if any(i == out for i in nxt.inputs[1:]):
                        break
                    chain.append(nxt)
                    cur = nxt
                if len(chain) < 2:
                    continue
                inputs = [chain[0].inputs[0]]
                ops, arity = [], []
                for n in chain:
                    ops.append(n.op_type)
                    arity.append(len(n.inputs))
                    inputs += n.inputs[1:]
                idx = graph.nodes.index(chain[-1])
                graph.add_node("FusedElementwise", inputs, [chain[-1].outputs[0]], {"ops": ops, "arity": arity},
                               name=f"fused_{chain[0].name or chain[0].id}", domain=RONN, index=idx)
                graph.remove_nodes([n.id for n in chain])
                stats.nodes_fused += len(chain) - 1
                progress = True
                break
        return stats

    @staticmethod
    def _elementwise(n, graph) -> bool:
        if n.attributes and n.op_type != "Gelu":
            return False
        if n.op_type == "Gelu" and n.attr("approximate", "none") != "tanh":
            return False                      # the fused chain evaluates the tanh form; the exact (Erf) form stays a node
        if n.op_type in _UNARY and len(n.inputs) == 1:
            return True
        return n.op_type in _BINARY and len(n.inputs) == 2 and all(i for i in n.inputs)

"""Tensor-parallel rewrite of an ONNX graph (Megatron layout), applied by a session created with ``tp_size > 1``.

The reference exercises "multi-GPU through session options" (benches/integration/multi_provider.rs:123-170) but its
providers pick one device per sub-graph; here every rank of a ``torch.distributed`` group builds the same session, and
this pass gives each rank its shard of the weights:

* MLP pairs  linear [K, F] -> element-wise activation(s) -> linear [F, N]: the first weight is split by columns, the
  second by rows (every rank holds F / world of the hidden features);
* attention  Q / K / V projections (fused or separate) -> Attention -> output linear: whole heads per rank, the output
  projection split by rows.

A ``com.ronn::AllReduce`` node after each row-parallel linear sums the partial results; its bias (and a fused residual)
stay on rank 0 only, so they are added once.  Everything that does not match stays replicated, which is correct, only
redundant.  The all-reduce runs on the session's process group (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ir import GraphNode, ModelGraph
from .base import OptimizationPass, PassStats

RONN = "com.ronn"
_LINEAR = ("MatMul", "Gemm", "FusedGemm")
_ELEMENTWISE = {"Relu", "Gelu", "FastGelu", "Tanh", "Sigmoid", "Identity", "Dropout", "Swish", "SiLU", "Erf"}


class TensorParallelPass(OptimizationPass):
    name = "TensorParallel"

    def __init__(self, rank: int, world: int):
        self.rank, self.world = int(rank), int(world)

    # ------------------------------------------------------------------ helpers
    def _linear(self, graph: ModelGraph, n: Optional[GraphNode]):
        """The [in, out] weight of a linear node with a constant weight, or None."""
        if n is None or n.op_type not in _LINEAR or len(n.inputs) < 2 or n.attr("tp"):
            return None
        w = graph.initializers.get(n.inputs[1])
        if w is None or w.dim() != 2 or not w.is_floating_point():
            return None
        if n.op_type == "Gemm" and (int(n.attr("transA", 0)) or float(n.attr("alpha", 1.0)) != 1.0
                                    or float(n.attr("beta", 1.0)) != 1.0):
            return None
        return w.t() if int(n.attr("transB", 0)) else w

    def _set_weight(self, graph: ModelGraph, n: GraphNode, w_in_out: torch.Tensor, tag: str) -> None:
        name = graph.fresh_name(f"{n.inputs[1]}.{tag}{self.rank}")
        graph.initializers[name] = w_in_out.contiguous()
        n.inputs[1] = name
        if n.op_type in ("Gemm", "FusedGemm"):
            n.attributes["transB"] = 0

    def _shard_bias(self, graph: ModelGraph, n: GraphNode, cols: torch.Tensor) -> bool:
        if len(n.inputs) > 2 and n.inputs[2]:
            b = graph.initializers.get(n.inputs[2])
            if b is None or b.dim() != 1:
                return False
            name = graph.fresh_name(f"{n.inputs[2]}.col{self.rank}")
            graph.initializers[name] = b[cols].contiguous()
            n.inputs[2] = name
        return True

    def _row_parallel(self, graph: ModelGraph, n: GraphNode, rows: torch.Tensor, w: torch.Tensor) -> None:
        """Second linear of a pair: rows of the weight, bias and fused residual on rank 0 only, all-reduce behind it."""
        self._set_weight(graph, n, w[rows, :], "row")
        if self.rank != 0:
            if len(n.inputs) > 2 and n.inputs[2]:
                b = graph.initializers[n.inputs[2]]
                name = graph.fresh_name(f"{n.inputs[2]}.zero")
                graph.initializers[name] = torch.zeros_like(b)
                n.inputs[2] = name
            if len(n.inputs) > 3:
                n.inputs = n.inputs[:3]                      # the fused residual is added by rank 0
        n.attributes["tp"] = "row"
        out = n.outputs[0]
        part = graph.fresh_name(out + ".partial")
        n.outputs[0] = part
        idx = graph.nodes.index(n) + 1
        graph.add_node("AllReduce", [part], [out], {}, name=f"{n.name or n.id}.all_reduce", domain=RONN, index=idx)

    def _range(self, total: int) -> Optional[torch.Tensor]:
        if total % self.world:
            return None
        per = total // self.world
        return torch.arange(self.rank * per, (self.rank + 1) * per)

    # ------------------------------------------------------------------ the pass
    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        if self.world <= 1:
            return stats
        outputs = set(graph.output_names())
        for n2 in list(graph.topological_order()):
            w2 = self._linear(graph, n2)
            if w2 is None or n2.attr("activation") or (len(n2.inputs) > 2 and n2.inputs[2]
                                                       and graph.initializers.get(n2.inputs[2]) is None):
                continue
            cons, prod = graph.consumers(), graph.producers()
            if self._mlp_pair(graph, n2, w2, cons, prod, outputs) or self._attention(graph, n2, w2, cons, prod, outputs):
                stats.nodes_modified += 1
        if stats.nodes_modified:
            graph.metadata["ronn.tp"] = f"{self.rank}/{self.world}"
            graph.sort_in_place()
        return stats

    def _mlp_pair(self, graph, n2, w2, cons, prod, outputs) -> bool:
        chain, cur = [], n2.inputs[0]
        while True:
            p = prod.get(cur)
            if p is None or cur in outputs or len(cons.get(cur, [])) != 1:
                return False
            if p.op_type in _ELEMENTWISE and len(p.inputs) == 1:
                chain.append(p)
                cur = p.inputs[0]
                continue
            break
        n1 = prod.get(cur)
        w1 = self._linear(graph, n1)
        if w1 is None or w1.shape[1] != w2.shape[0] or len(n1.inputs) > 3 or n1 is n2:
            return False
        cols = self._range(w1.shape[1])
        if cols is None:
            return False
        if len(n1.inputs) > 2 and n1.inputs[2] and graph.initializers.get(n1.inputs[2]) is None:
            return False
        if not self._shard_bias(graph, n1, cols):
            return False
        self._set_weight(graph, n1, w1[:, cols], "col")
        n1.attributes["tp"] = "col"
        self._row_parallel(graph, n2, cols, w2)
        return True

    def _attention(self, graph, n2, w2, cons, prod, outputs) -> bool:
        att = prod.get(n2.inputs[0])
        if att is None or att.op_type not in ("Attention", "MultiHeadAttention") or len(cons.get(att.outputs[0], [])) != 1:
            return False
        heads = int(att.attr("num_heads", 0))
        H = w2.shape[0]
        if heads <= 0 or heads % self.world or H % heads:
            return False
        d = H // heads
        hcols = torch.arange(self.rank * (heads // self.world) * d, (self.rank + 1) * (heads // self.world) * d)
        srcs = [prod.get(t) for t in att.inputs[:3]]
        if any(s is None for s in srcs):
            return False
        if len({s.id for s in srcs}) == 1 and srcs[0].op_type == "Split":
            # fused projection [K, 3H] -> Split: take this rank's heads out of each third
            sp = srcs[0]
            proj = prod.get(sp.inputs[0])
            w = self._linear(graph, proj)
            sizes = graph.initializers.get(sp.inputs[1]) if len(sp.inputs) > 1 else None
            if w is None or sizes is None or sizes.tolist() != [H, H, H] or w.shape[1] != 3 * H or len(cons.get(proj.outputs[0], [])) != 1:
                return False
            cols = torch.cat([hcols, H + hcols, 2 * H + hcols])
            if not self._shard_bias(graph, proj, cols):
                return False
            self._set_weight(graph, proj, w[:, cols], "col")
            proj.attributes["tp"] = "col"
            name = graph.fresh_name(sp.inputs[1] + f".tp{self.rank}")
            graph.initializers[name] = torch.tensor([hcols.numel()] * 3, dtype=torch.int64)
            sp.inputs[1] = name
        else:
            ws = [self._linear(graph, s) for s in srcs]
            if any(w is None or w.shape[1] != H for w in ws) or len({s.id for s in srcs}) != 3:
                return False
            if any(len(cons.get(s.outputs[0], [])) != 1 or len(s.inputs) > 3 or s.attr("activation") for s in srcs):
                return False
            for s, w in zip(srcs, ws):
                if not self._shard_bias(graph, s, hcols):
                    return False
                self._set_weight(graph, s, w[:, hcols], "col")
                s.attributes["tp"] = "col"
        att.attributes["num_heads"] = heads // self.world
        self._row_parallel(graph, n2, hcols, w2)
        return True

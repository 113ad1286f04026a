"""Dead-code elimination by backward reachability from the graph outputs.

(The reference marks every node live and never mutates:
crates/ronn-graph/src/passes/dead_code.rs:15-50.)  Unused initializers are dropped too.
"""
from __future__ import annotations

from ..ir import ModelGraph
from .base import OptimizationPass, PassStats


class DeadCodeEliminationPass(OptimizationPass):
    name = "DeadCodeElimination"

    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        if graph.nodes:
            live = graph.live_node_ids()
            dead = [n.id for n in graph.nodes if n.id not in live]
            if dead:
                stats.nodes_removed = graph.remove_nodes(dead)
        used = {i for n in graph.nodes for i in n.inputs if i} | set(graph.output_names())
        for name in [k for k in graph.initializers if k not in used]:
            del graph.initializers[name]
        return stats

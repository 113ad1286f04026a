"""Pass interface (crates/ronn-graph/src/passes/mod.rs:20-31)."""
from __future__ import annotations

from dataclasses import dataclass

from ..ir import ModelGraph


@dataclass
class PassStats:
    nodes_removed: int = 0
    nodes_fused: int = 0
    nodes_modified: int = 0

    @property
    def changed(self) -> bool:
        return bool(self.nodes_removed or self.nodes_fused or self.nodes_modified)


class OptimizationPass:
    name = "Pass"

    def run(self, graph: ModelGraph) -> PassStats:          # pragma: no cover - interface
        raise NotImplementedError

    def should_run(self, graph: ModelGraph) -> bool:
        return True

"""Optimisation pipeline.

Levels as in the reference (crates/ronn-graph/src/optimizer.rs:8-60): O0 none; O1
ConstantFolding + DeadCodeElimination; O2 adds NodeFusion + LayoutOptimization; O3 adds
CpuOptimization + GpuOptimization.  The pass manager repeats the list until no pass reports a
change, at most 10 iterations (optimizer.rs:96-138).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from ..api.errors import OptimizationError
from ..core.types import OptimizationLevel, ProviderType
from .ir import ModelGraph
from .passes.base import OptimizationPass, PassStats
from .passes.constant_folding import ConstantFoldingPass
from .passes.dead_code import DeadCodeEliminationPass
from .passes.fusion import NodeFusionPass
from .passes.layout import LayoutOptimizationPass
from .passes.provider_specific import CpuOptimizationPass, GpuOptimizationPass

MAX_ITERATIONS = 10


@dataclass
class OptimizationStats:
    nodes_removed: int = 0
    nodes_fused: int = 0
    nodes_modified: int = 0
    iterations: int = 0

    def merge(self, s: PassStats) -> None:
        self.nodes_removed += s.nodes_removed
        self.nodes_fused += s.nodes_fused
        self.nodes_modified += s.nodes_modified

    def total_changes(self) -> int:
        return self.nodes_removed + self.nodes_fused + self.nodes_modified


class PassManager:
    def __init__(self):
        self.passes: List[OptimizationPass] = []

    def add_pass(self, p: OptimizationPass) -> None:
        self.passes.append(p)

    def pass_count(self) -> int:
        return len(self.passes)

    def run(self, graph: ModelGraph) -> OptimizationStats:
        total = OptimizationStats()
        for it in range(MAX_ITERATIONS):
            total.iterations = it + 1
            changed = False
            for p in self.passes:
                if not p.should_run(graph):
                    continue
                try:
                    s = p.run(graph)
                except Exception as e:                      # a broken pass must not corrupt the session silently
                    raise OptimizationError(f"pass {p.name} failed: {e}") from e
                total.merge(s)
                changed = changed or s.changed
            if not changed:
                break
        return total


class Optimizer:
    def __init__(self, level: OptimizationLevel = OptimizationLevel.O2, provider: Optional[ProviderType] = None):
        self.level = OptimizationLevel.parse(level)
        self.provider = provider
        self.manager = PassManager()
        if self.level >= OptimizationLevel.O1:
            self.manager.add_pass(ConstantFoldingPass())
            self.manager.add_pass(DeadCodeEliminationPass())
        if self.level >= OptimizationLevel.O2:
            self.manager.add_pass(NodeFusionPass())
            self.manager.add_pass(LayoutOptimizationPass())
        if self.level >= OptimizationLevel.O3:
            cpu, gpu = CpuOptimizationPass(), GpuOptimizationPass()
            # both are registered (pass_count stays 6); each only acts for its own provider when one is known
            if provider is not None:
                cpu.should_run = lambda g, _p=provider: _p == ProviderType.CPU
                gpu.should_run = lambda g, _p=provider: _p in (ProviderType.GPU, ProviderType.BITNET)
            else:
                gpu.should_run = lambda g: False
            self.manager.add_pass(cpu)
            self.manager.add_pass(gpu)

    def pass_count(self) -> int:
        return self.manager.pass_count()

    def pass_names(self) -> List[str]:
        return [p.name for p in self.manager.passes]

    def optimize(self, graph: ModelGraph) -> OptimizationStats:
        return self.manager.run(graph)

"""``HierarchicalReasoningModule`` (crates/ronn-hrm/src/lib.rs:53-201): assess -> route -> execute;
Hybrid runs System 1 and returns System 2's result when uncertainty > 0.5."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

from .complexity import ComplexityMetrics
from .executor import ExecutionPath, HighLevelPlanner, LowLevelExecutor
from .router import HRMRouter, RoutingStrategy


@dataclass
class ProcessingResult:
    output: Any
    path_taken: ExecutionPath
    complexity_metrics: ComplexityMetrics
    confidence: float


@dataclass
class HRMMetrics:
    system1_count: int = 0
    system2_count: int = 0
    hybrid_count: int = 0

    @property
    def total(self) -> int:
        return self.system1_count + self.system2_count + self.hybrid_count

    def percentages(self):
        t = self.total or 1
        return (100.0 * self.system1_count / t, 100.0 * self.system2_count / t, 100.0 * self.hybrid_count / t)


class HierarchicalReasoningModule:
    def __init__(self, strategy: RoutingStrategy = RoutingStrategy.ADAPTIVE_COMPLEXITY,
                 system1: Optional[Callable] = None, system2: Optional[Callable] = None):
        self.router = HRMRouter(strategy)
        self.low = LowLevelExecutor(system1)
        self.high = HighLevelPlanner(system2)
        self._metrics = HRMMetrics()

    @staticmethod
    def with_strategy(strategy: RoutingStrategy) -> "HierarchicalReasoningModule":
        return HierarchicalReasoningModule(strategy)

    def process(self, x, payload=None) -> ProcessingResult:
        """``x`` is the tensor whose complexity decides the route; ``payload`` (default ``x``) is what the
        executors receive."""
        m = self.router.assess_complexity(x)
        d = self.router.route(m)
        arg = x if payload is None else payload
        if d.path == ExecutionPath.SYSTEM1:
            out = self.low.execute(arg)
            self._metrics.system1_count += 1
        elif d.path == ExecutionPath.SYSTEM2:
            out = self.high.execute(arg)
            self._metrics.system2_count += 1
        else:
            out = self.low.execute(arg)
            if m.uncertainty > 0.5:
                out = self.high.execute(arg)
            self._metrics.hybrid_count += 1
        return ProcessingResult(out, d.path, m, d.confidence)

    def metrics(self) -> HRMMetrics:
        return self._metrics

    def reset_metrics(self) -> None:
        self._metrics = HRMMetrics()

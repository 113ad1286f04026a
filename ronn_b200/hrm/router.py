"""Routing (crates/ronn-hrm/src/router.rs:12-197): Low -> System1, High -> System2, Medium -> Hybrid when
allowed and uncertain (> 0.6) else System1 "favoring speed" with confidence 0.6."""
from __future__ import annotations

import enum
from dataclasses import dataclass

from .complexity import ComplexityAssessor, ComplexityLevel, ComplexityMetrics
from .executor import ExecutionPath


class RoutingStrategy(enum.Enum):
    ALWAYS_SYSTEM1 = "always_system1"
    ALWAYS_SYSTEM2 = "always_system2"
    ADAPTIVE_COMPLEXITY = "adaptive_complexity"
    ADAPTIVE_HYBRID = "adaptive_hybrid"


@dataclass
class RoutingDecision:
    path: ExecutionPath
    confidence: float
    reason: str


@dataclass
class RouterStats:
    total_routes: int = 0
    system1_routes: int = 0
    system2_routes: int = 0
    hybrid_routes: int = 0

    def _pct(self, n: int) -> float:
        return 100.0 * n / self.total_routes if self.total_routes else 0.0

    @property
    def system1_percentage(self) -> float:
        return self._pct(self.system1_routes)

    @property
    def system2_percentage(self) -> float:
        return self._pct(self.system2_routes)

    @property
    def hybrid_percentage(self) -> float:
        return self._pct(self.hybrid_routes)


class HRMRouter:
    def __init__(self, strategy: RoutingStrategy = RoutingStrategy.ADAPTIVE_COMPLEXITY, assessor: ComplexityAssessor = None):
        self.strategy = strategy
        self.assessor = assessor or ComplexityAssessor()
        self.stats = RouterStats()

    def set_strategy(self, strategy: RoutingStrategy) -> None:
        self.strategy = strategy

    def assess_complexity(self, x) -> ComplexityMetrics:
        return self.assessor.assess(x)

    def route(self, m: ComplexityMetrics) -> RoutingDecision:
        if self.strategy == RoutingStrategy.ALWAYS_SYSTEM1:
            d = RoutingDecision(ExecutionPath.SYSTEM1, 1.0, "strategy: always System 1")
        elif self.strategy == RoutingStrategy.ALWAYS_SYSTEM2:
            d = RoutingDecision(ExecutionPath.SYSTEM2, 1.0, "strategy: always System 2")
        else:
            d = self._adaptive(m, self.strategy == RoutingStrategy.ADAPTIVE_HYBRID)
        self.stats.total_routes += 1
        if d.path == ExecutionPath.SYSTEM1:
            self.stats.system1_routes += 1
        elif d.path == ExecutionPath.SYSTEM2:
            self.stats.system2_routes += 1
        else:
            self.stats.hybrid_routes += 1
        return d

    @staticmethod
    def _adaptive(m: ComplexityMetrics, allow_hybrid: bool) -> RoutingDecision:
        if m.level == ComplexityLevel.LOW:
            return RoutingDecision(ExecutionPath.SYSTEM1, 1.0 - m.uncertainty, "low complexity: fast path")
        if m.level == ComplexityLevel.HIGH:
            return RoutingDecision(ExecutionPath.SYSTEM2, 1.0 - m.uncertainty, "high complexity: precise path")
        if allow_hybrid and m.uncertainty > 0.6:
            return RoutingDecision(ExecutionPath.HYBRID, 0.5, "medium complexity, uncertain: hybrid")
        return RoutingDecision(ExecutionPath.SYSTEM1, 0.6, "medium complexity: favoring speed")

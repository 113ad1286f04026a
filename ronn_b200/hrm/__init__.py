"""Hierarchical Reasoning Module: complexity assessment and routing between a fast (BitNet) path and
a precise (full-precision) path (crates/ronn-hrm/src/lib.rs:53-201)."""
from .complexity import ComplexityAssessor, ComplexityLevel, ComplexityMetrics
from .executor import ExecutionPath, HighLevelPlanner, LowLevelExecutor
from .module import HierarchicalReasoningModule, HRMMetrics, ProcessingResult
from .router import HRMRouter, RouterStats, RoutingDecision, RoutingStrategy

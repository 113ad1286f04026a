"""Complexity assessment (crates/ronn-hrm/src/complexity.rs:10-148).

score = min(0.5*size + 0.3*variance + 0.2*dim, 1) with size linear between 100 and 1000 elements,
variance = population variance / max(2*0.5, 1), dim = min(ndim/4, 1); level Low < 0.33 <= Medium
< 0.66 <= High; uncertainty 0.8 for Medium, 0.2 otherwise.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class ComplexityLevel(enum.Enum):
    LOW = "low"
    MEDIUM = "medium"
    HIGH = "high"


@dataclass
class ComplexityMetrics:
    level: ComplexityLevel
    size: int
    variance: float
    dimensionality: int
    uncertainty: float
    complexity_score: float


class ComplexityAssessor:
    def __init__(self, low_threshold: int = 100, high_threshold: int = 1000, variance_threshold: float = 0.5):
        self.low_threshold = low_threshold
        self.high_threshold = high_threshold
        self.variance_threshold = variance_threshold

    def assess(self, x: torch.Tensor) -> ComplexityMetrics:
        size = int(x.numel())
        if size:
            xf = x.detach().float()
            variance = float(xf.var(unbiased=False)) if size > 1 else 0.0
        else:
            variance = 0.0
        ndim = x.dim()
        if size < self.low_threshold:
            size_score = 0.0
        elif size > self.high_threshold:
            size_score = 1.0
        else:
            size_score = (size - self.low_threshold) / float(self.high_threshold - self.low_threshold)
        variance_score = variance / max(2.0 * self.variance_threshold, 1.0)
        dim_score = min(ndim / 4.0, 1.0)
        score = min(0.5 * size_score + 0.3 * variance_score + 0.2 * dim_score, 1.0)
        level = ComplexityLevel.LOW if score < 0.33 else (ComplexityLevel.MEDIUM if score < 0.66 else ComplexityLevel.HIGH)
        uncertainty = 0.8 if level == ComplexityLevel.MEDIUM else 0.2
        return ComplexityMetrics(level, size, variance, ndim, uncertainty, score)

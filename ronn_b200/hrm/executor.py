"""Executors of the two paths (crates/ronn-hrm/src/executor.rs:12-176).

In the reference both executors return ``input.clone()``.  Here each wraps a callable - by default
identity, in a routed session the BitNet session (System 1) and the full-precision session
(System 2)."""
from __future__ import annotations

import enum
import time
from typing import Callable, Optional


class ExecutionPath(enum.Enum):
    SYSTEM1 = "system1"
    SYSTEM2 = "system2"
    HYBRID = "hybrid"


class _Executor:
    label = ""

    def __init__(self, fn: Optional[Callable] = None):
        self.fn = fn
        self.execution_count = 0
        self.total_time_us = 0.0

    def execute(self, x):
        t = time.perf_counter()
        y = self.fn(x) if self.fn is not None else (x.clone() if hasattr(x, "clone") else x)
        self.execution_count += 1
        self.total_time_us += (time.perf_counter() - t) * 1e6
        return y


class LowLevelExecutor(_Executor):
    """System 1: fast, approximate (BitNet)."""
    label = "System1"


class HighLevelPlanner(_Executor):
    """System 2: slow, precise (full precision)."""
    label = "System2"

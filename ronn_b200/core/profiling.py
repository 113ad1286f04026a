"""In-process profiler (crates/ronn-core/src/profiling.rs:12-423).

RAII-style scopes produce ``ProfileEvent{name, category, duration_us, metadata}``; reports
aggregate by category and by name (count, total, avg, min, max, std) and export JSON and
Chrome-trace JSON.  On CUDA devices a scope is timed with CUDA events on the current stream
(device time, resolved lazily when the report is built), which the reference does not have;
and unlike the reference (where ``enable_profiling`` is dead: crates/ronn-api/src/session.rs:18)
the session's executor opens one scope per node.
"""
from __future__ import annotations

import json
import math
import threading
import os
import time
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class ProfileConfig:
    enabled: bool = True
    profile_ops: bool = True
    profile_memory: bool = False
    profile_transfers: bool = False
    min_duration_us: float = 0.0

    @staticmethod
    def development() -> "ProfileConfig":
        return ProfileConfig(True, True, True, True, 0.0)

    @staticmethod
    def production() -> "ProfileConfig":
        return ProfileConfig(True, True, False, False, 100.0)

    @staticmethod
    def disabled() -> "ProfileConfig":
        return ProfileConfig(False, False, False, False, 0.0)


@dataclass
class ProfileEvent:
    name: str
    category: str
    duration_us: float
    start_us: float = 0.0
    metadata: Dict[str, str] = field(default_factory=dict)


@dataclass
class AggregateStats:
    count: int
    total_us: float
    avg_us: float
    min_us: float
    max_us: float
    std_us: float


def _aggregate(durs: List[float]) -> AggregateStats:
    n = len(durs)
    total = sum(durs)
    avg = total / n
    var = sum((d - avg) ** 2 for d in durs) / n
    return AggregateStats(n, total, avg, min(durs), max(durs), math.sqrt(var))


class ProfileReport:
    def __init__(self, events: List[ProfileEvent]):
        self.events = events
        self.total_us = sum(e.duration_us for e in events)
        self.by_category: Dict[str, AggregateStats] = {}
        self.by_name: Dict[str, AggregateStats] = {}
        cat: Dict[str, List[float]] = {}
        nam: Dict[str, List[float]] = {}
        for e in events:
            cat.setdefault(e.category, []).append(e.duration_us)
            nam.setdefault(e.name, []).append(e.duration_us)
        self.by_category = {k: _aggregate(v) for k, v in cat.items()}
        self.by_name = {k: _aggregate(v) for k, v in nam.items()}

    def to_json(self) -> str:
        def enc(d):
            return {k: vars(v) for k, v in d.items()}
        return json.dumps({"total_us": self.total_us, "event_count": len(self.events),
                           "by_category": enc(self.by_category), "by_name": enc(self.by_name)}, indent=2)

    def to_chrome_trace(self) -> str:
        return json.dumps({"traceEvents": [
            {"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": e.duration_us, "pid": 0, "tid": 0,
             "args": e.metadata} for e in self.events]})

    def print(self) -> None:
        print(f"=== profile: {len(self.events)} events, {self.total_us / 1e3:.3f} ms total ===")
        for k, s in sorted(self.by_category.items(), key=lambda kv: -kv[1].total_us):
            print(f"  [{k}] n={s.count} total={s.total_us / 1e3:.3f} ms avg={s.avg_us:.1f} us")
        for k, s in sorted(self.by_name.items(), key=lambda kv: -kv[1].total_us)[:20]:
            print(f"    {k}: n={s.count} total={s.total_us / 1e3:.3f} ms avg={s.avg_us:.1f} us "
                  f"min={s.min_us:.1f} max={s.max_us:.1f} std={s.std_us:.1f}")


class Profiler:
    def __init__(self, config: Optional[ProfileConfig] = None):
        self.config = config or ProfileConfig()
        self._lock = threading.Lock()
        self._events: List[ProfileEvent] = []
        self._pending = []           # (name, category, start_us, start_event, end_event, metadata)
        self._t0 = time.perf_counter()

    @property
    def enabled(self) -> bool:
        return self.config.enabled

    def record(self, event: ProfileEvent) -> None:
        if not self.config.enabled or event.duration_us < self.config.min_duration_us:
            return
        with self._lock:
            self._events.append(event)

    @contextmanager
    def scope(self, name: str, category: str = "op", device=None, **metadata):
        if not self.config.enabled:
            yield
            return
        start = (time.perf_counter() - self._t0) * 1e6
        if device is not None and getattr(device, "type", "cpu") == "cuda":
            import torch
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            nvtx = os.environ.get("RONN_NVTX", "0") == "1"       # named ranges for external timeline tools
            if nvtx:
                torch.cuda.nvtx.range_push(f"{category}:{name}")
            e0.record()
            try:
                yield
            finally:
                e1.record()
                if nvtx:
                    torch.cuda.nvtx.range_pop()
                with self._lock:
                    self._pending.append((name, category, start, e0, e1, {k: str(v) for k, v in metadata.items()}))
        else:
            t = time.perf_counter()
            try:
                yield
            finally:
                self.record(ProfileEvent(name, category, (time.perf_counter() - t) * 1e6, start,
                                         {k: str(v) for k, v in metadata.items()}))

    def _resolve_pending(self):
        with self._lock:
            pend, self._pending = self._pending, []
        if not pend:
            return
        import torch
        torch.cuda.synchronize()
        for name, cat, start, e0, e1, md in pend:
            self.record(ProfileEvent(name, cat, e0.elapsed_time(e1) * 1e3, start, md))

    def events(self) -> List[ProfileEvent]:
        self._resolve_pending()
        with self._lock:
            return list(self._events)

    def report(self) -> ProfileReport:
        return ProfileReport(self.events())

    def clear(self) -> None:
        self._resolve_pending()
        with self._lock:
            self._events.clear()


_GLOBAL: Optional[Profiler] = None


def init_profiler(config: Optional[ProfileConfig] = None) -> Profiler:
    global _GLOBAL
    _GLOBAL = Profiler(config)
    return _GLOBAL


def global_profiler() -> Profiler:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = Profiler(ProfileConfig.disabled())
    return _GLOBAL


@contextmanager
def profile(name: str, category: str = "op", **metadata):
    with global_profiler().scope(name, category, **metadata):
        yield

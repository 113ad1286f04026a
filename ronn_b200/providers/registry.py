"""Provider registry (crates/ronn-providers/src/registry.rs:16-310).

Preference order by performance profile (GPU first, then CPU, memory-optimised,
power-efficient), ``select_provider`` = first provider that supports every op,
``get_fallback_chain`` = greedy per-op assignment in preference order.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from ..api.errors import ProviderError
from ..core.types import OperatorSpec, PerformanceProfile, ProviderCapability, ProviderType
from ..graph.ir import SubGraph
from .base import ExecutionProvider

_PROFILE_RANK = {PerformanceProfile.GPU: 0, PerformanceProfile.CPU: 1, PerformanceProfile.MEMORY_OPTIMIZED: 2,
                 PerformanceProfile.POWER_EFFICIENT: 3}


@dataclass
class RegistryStatistics:
    provider_count: int
    total_supported_ops: int
    preference_order: List[ProviderType]


class ProviderRegistry:
    def __init__(self):
        self._lock = threading.RLock()
        self._providers: Dict[ProviderType, ExecutionProvider] = {}
        self._caps: Dict[ProviderType, ProviderCapability] = {}
        self._order: List[ProviderType] = []

    def register_provider(self, provider: ExecutionProvider) -> None:
        with self._lock:
            pid = provider.provider_id
            if pid in self._providers:
                raise ProviderError(f"Provider {pid.name} is already registered")
            self._providers[pid] = provider
            self._caps[pid] = provider.get_capability()
            self._order.append(pid)
            self._order.sort(key=lambda p: _PROFILE_RANK[self._caps[p].performance_profile])

    def unregister_provider(self, pid: ProviderType) -> None:
        with self._lock:
            if pid not in self._providers:
                raise ProviderError(f"Provider {pid.name} is not registered")
            self._providers.pop(pid).shutdown()
            self._caps.pop(pid)
            self._order.remove(pid)

    def get_provider(self, pid: ProviderType) -> Optional[ExecutionProvider]:
        with self._lock:
            return self._providers.get(pid)

    def get_capability(self, pid: ProviderType) -> Optional[ProviderCapability]:
        with self._lock:
            return self._caps.get(pid)

    def get_provider_ids(self) -> List[ProviderType]:
        with self._lock:
            return list(self._order)

    def provider_count(self) -> int:
        with self._lock:
            return len(self._providers)

    def set_preference_order(self, order: Sequence[ProviderType]) -> None:
        with self._lock:
            for p in order:
                if p not in self._providers:
                    raise ProviderError(f"Provider {p.name} in preference order is not registered")
            rest = [p for p in self._order if p not in order]
            self._order = list(order) + rest

    def get_preference_order(self) -> List[ProviderType]:
        with self._lock:
            return list(self._order)

    def select_provider(self, ops: Sequence[OperatorSpec]) -> Optional[ProviderType]:
        with self._lock:
            for pid in self._order:
                if all(self._providers[pid].can_handle(ops)):
                    return pid
            return None

    def get_fallback_chain(self, ops: Sequence[OperatorSpec]) -> List[Tuple[OperatorSpec, Optional[ProviderType]]]:
        with self._lock:
            out = []
            for o in ops:
                chosen = None
                for pid in self._order:
                    if self._providers[pid].can_handle([o])[0]:
                        chosen = pid
                        break
                out.append((o, chosen))
            return out

    def compile_subgraph(self, subgraph: SubGraph, initializers=None):
        specs = [OperatorSpec(n.op_type) for n in subgraph.nodes]
        pid = self.select_provider(specs)
        if pid is None:
            raise ProviderError("no registered provider supports every operator of the subgraph: "
                                + ", ".join(sorted({s.op_type for s in specs})))
        return pid, self._providers[pid].compile_subgraph(subgraph, initializers)

    def get_statistics(self) -> RegistryStatistics:
        with self._lock:
            ops = set()
            for c in self._caps.values():
                ops |= set(c.supported_ops)
            return RegistryStatistics(len(self._providers), len(ops), list(self._order))

    def shutdown(self) -> None:
        with self._lock:
            for p in list(self._providers.values()):
                p.shutdown()
            self._providers.clear()
            self._caps.clear()
            self._order.clear()

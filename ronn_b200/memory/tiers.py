"""Working / episodic / semantic memory and sleep consolidation.

Behaviour of the reference modules: working memory with capacity 100, TTL 60 s and FIFO / LRU
eviction (crates/ronn-memory/src/working.rs:9-125); episodic store with a temporal index and
``EpisodeQuery`` (episodic.rs:9-101); concept graph with spreading activation at half strength
(semantic.rs:8-133); consolidation of important episodes into ``Pattern_i`` concepts with ids offset
by 10000 (consolidation.rs:9-105); ``MultiTierMemory`` routing (lib.rs:60-158).  ``search_similar``
ranks by cosine similarity of the stored tensors (the reference returns the most recent items).
"""
from __future__ import annotations

import bisect
import enum
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


class EvictionPolicy(enum.Enum):
    FIFO = "fifo"
    LRU = "lru"


@dataclass
class WorkingMemoryConfig:
    capacity: int = 100
    ttl_seconds: float = 60.0
    eviction: EvictionPolicy = EvictionPolicy.LRU


@dataclass
class MemoryItem:
    id: int
    data: torch.Tensor
    importance: float
    timestamp: float
    last_access: float


class WorkingMemory:
    def __init__(self, config: WorkingMemoryConfig = None):
        self.config = config or WorkingMemoryConfig()
        self._items: "OrderedDict[int, MemoryItem]" = OrderedDict()
        self._next = 1

    def __len__(self):
        return len(self._items)

    def store(self, data: torch.Tensor, importance: float = 0.5) -> int:
        now = time.time()
        while len(self._items) >= self.config.capacity:
            self._items.popitem(last=False)
        i = self._next
        self._next += 1
        self._items[i] = MemoryItem(i, data, float(importance), now, now)
        return i

    def get(self, item_id: int) -> Optional[MemoryItem]:
        it = self._items.get(item_id)
        if it is not None:
            it.last_access = time.time()
            if self.config.eviction == EvictionPolicy.LRU:
                self._items.move_to_end(item_id)
        return it

    def search_similar(self, query: torch.Tensor, k: int = 5) -> List[MemoryItem]:
        q = query.detach().float().reshape(-1)
        scored = []
        for it in self._items.values():
            d = it.data.detach().float().reshape(-1)
            if d.numel() == q.numel() and q.numel():
                s = float(torch.nn.functional.cosine_similarity(q, d, dim=0))
            else:
                s = -1.0
            scored.append((s, it.timestamp, it))
        scored.sort(key=lambda t: (t[0], t[1]), reverse=True)
        return [it for _, _, it in scored[:k]]

    def drain_old_items(self, now: Optional[float] = None) -> List[MemoryItem]:
        now = time.time() if now is None else now
        old = [i for i, it in self._items.items() if now - it.timestamp > self.config.ttl_seconds]
        return [self._items.pop(i) for i in old]

    def items(self) -> List[MemoryItem]:
        return list(self._items.values())


@dataclass
class Episode:
    id: int
    data: torch.Tensor
    timestamp: float
    importance: float


@dataclass
class EpisodeQuery:
    start: Optional[float] = None
    end: Optional[float] = None
    min_importance: Optional[float] = None
    limit: Optional[int] = None


class EpisodicMemory:
    def __init__(self):
        self._episodes: Dict[int, Episode] = {}
        self._index: List[Tuple[float, int]] = []
        self._next = 1

    def __len__(self):
        return len(self._episodes)

    def store(self, data: torch.Tensor, importance: float, timestamp: Optional[float] = None) -> int:
        ts = time.time() if timestamp is None else timestamp
        i = self._next
        self._next += 1
        self._episodes[i] = Episode(i, data, ts, float(importance))
        bisect.insort(self._index, (ts, i))
        return i

    def get(self, episode_id: int) -> Optional[Episode]:
        return self._episodes.get(episode_id)

    def query(self, q: EpisodeQuery) -> List[Episode]:
        out = []
        for ts, i in self._index:
            if q.start is not None and ts < q.start:
                continue
            if q.end is not None and ts > q.end:
                break
            e = self._episodes[i]
            if q.min_importance is not None and e.importance < q.min_importance:
                continue
            out.append(e)
            if q.limit is not None and len(out) >= q.limit:
                break
        return out

    def all(self) -> List[Episode]:
        return [self._episodes[i] for _, i in self._index]


@dataclass
class Concept:
    id: int
    name: str
    activation: float = 0.0


class ConceptGraph:
    def __init__(self):
        self.concepts: Dict[int, Concept] = {}
        self.edges: Dict[int, Dict[int, float]] = {}

    def add_concept(self, c: Concept) -> None:
        self.concepts[c.id] = c
        self.edges.setdefault(c.id, {})

    def add_relationship(self, a: int, b: int, weight: float = 1.0) -> None:
        if a not in self.concepts or b not in self.concepts:
            raise KeyError("both concepts must exist")
        self.edges[a][b] = weight
        self.edges[b][a] = weight

    def activate(self, concept_id: int, amount: float) -> None:
        c = self.concepts.get(concept_id)
        if c is None:
            return
        c.activation += amount
        for nb, w in self.edges.get(concept_id, {}).items():
            self.concepts[nb].activation += 0.5 * amount * w

    def neighbours(self, concept_id: int) -> List[int]:
        return list(self.edges.get(concept_id, {}))


class SemanticMemory:
    def __init__(self):
        self.graph = ConceptGraph()

    def __len__(self):
        return len(self.graph.concepts)

    def store_concept(self, c: Concept) -> None:
        self.graph.add_concept(c)

    def relate(self, a: int, b: int, weight: float = 1.0) -> None:
        self.graph.add_relationship(a, b, weight)

    def activate(self, concept_id: int, amount: float = 1.0) -> None:
        self.graph.activate(concept_id, amount)

    def get(self, concept_id: int) -> Optional[Concept]:
        return self.graph.concepts.get(concept_id)


@dataclass
class ConsolidationConfig:
    importance_threshold: float = 0.5
    max_patterns_per_cycle: int = 10


@dataclass
class ConsolidationResult:
    episodes_considered: int
    patterns_created: int


class SleepConsolidation:
    def __init__(self, config: ConsolidationConfig = None):
        self.config = config or ConsolidationConfig()
        self.cycles = 0

    def consolidate(self, episodic: EpisodicMemory, semantic: SemanticMemory) -> ConsolidationResult:
        important = [e for e in episodic.all() if e.importance >= self.config.importance_threshold]
        important.sort(key=lambda e: -e.importance)
        made = 0
        for k, e in enumerate(important[: self.config.max_patterns_per_cycle]):
            cid = e.id + 10000
            if semantic.get(cid) is None:
                semantic.store_concept(Concept(cid, f"Pattern_{k}"))
                made += 1
        self.cycles += 1
        return ConsolidationResult(len(important), made)


@dataclass
class MemoryStats:
    working_count: int
    episodic_count: int
    semantic_count: int
    consolidation_cycles: int


class MultiTierMemory:
    def __init__(self, working: WorkingMemoryConfig = None, consolidation: ConsolidationConfig = None):
        self.working = WorkingMemory(working)
        self.episodic = EpisodicMemory()
        self.semantic = SemanticMemory()
        self.consolidator = SleepConsolidation(consolidation)

    def store(self, data: torch.Tensor, importance: float = 0.5) -> int:
        i = self.working.store(data, importance)
        if importance > 0.7:
            self.episodic.store(data, importance)
        return i

    def retrieve(self, item_id: int) -> Optional[torch.Tensor]:
        it = self.working.get(item_id)
        return None if it is None else it.data

    def search_similar(self, query: torch.Tensor, k: int = 5) -> List[MemoryItem]:
        return self.working.search_similar(query, k)

    async def consolidate(self) -> ConsolidationResult:
        return self.consolidate_sync()

    def consolidate_sync(self, now: Optional[float] = None) -> ConsolidationResult:
        for it in self.working.drain_old_items(now):
            if it.importance > 0.5:
                self.episodic.store(it.data, it.importance, it.timestamp)
        return self.consolidator.consolidate(self.episodic, self.semantic)

    def stats(self) -> MemoryStats:
        return MemoryStats(len(self.working), len(self.episodic), len(self.semantic), self.consolidator.cycles)

"""Multi-tier memory: working, episodic, semantic, consolidation (crates/ronn-memory/src/lib.rs:60-158)."""
from .tiers import (Concept, ConceptGraph, ConsolidationConfig, Episode, EpisodeQuery, EpisodicMemory, MemoryItem,
                    MemoryStats, MultiTierMemory, SemanticMemory, SleepConsolidation, WorkingMemory,
                    WorkingMemoryConfig)

"""Memory tiers, continual learning and hierarchical routing, one behaviour per test (the reference keeps these as unit
tests beside each module: crates/ronn-memory/src/{working,episodic,semantic,consolidation}.rs,
crates/ronn-learning/src/{timescales,ewc,replay}.rs, crates/ronn-hrm/src/{complexity,router,executor}.rs)."""
import asyncio

import pytest
import torch

from ronn_b200.hrm.complexity import ComplexityAssessor, ComplexityLevel
from ronn_b200.hrm.executor import ExecutionPath
from ronn_b200.hrm.module import HierarchicalReasoningModule
from ronn_b200.hrm.router import HRMRouter, RoutingStrategy
from ronn_b200.learning.engine import (ContinualLearningEngine, ElasticWeightConsolidation, Experience, ExperienceReplay,
                                       LearningConfig, MultiTimescaleLearner, ReplayStrategy, TimescaleConfig)
from ronn_b200.memory.tiers import (Concept, ConceptGraph, ConsolidationConfig, EpisodeQuery, EpisodicMemory, EvictionPolicy,
                                    MultiTierMemory, SemanticMemory, SleepConsolidation, WorkingMemory, WorkingMemoryConfig)


# ---------------------------------------------------------------------------------------------- working memory
def test_working_memory_assigns_increasing_ids_and_returns_what_was_stored():
    wm = WorkingMemory()
    a, b = wm.store(torch.tensor([1.0, 2.0]), 0.3), wm.store(torch.tensor([3.0]), 0.9)
    assert b == a + 1 and len(wm) == 2
    assert wm.get(a).data.tolist() == [1.0, 2.0] and wm.get(b).importance == pytest.approx(0.9)
    assert wm.get(12345) is None


@pytest.mark.parametrize("capacity", [1, 3, 10])
def test_working_memory_never_exceeds_its_capacity(capacity):
    wm = WorkingMemory(WorkingMemoryConfig(capacity=capacity))
    ids = [wm.store(torch.tensor([float(i)])) for i in range(capacity + 5)]
    assert len(wm) == capacity
    assert [it.id for it in wm.items()] == ids[-capacity:]            # the oldest were dropped


def test_fifo_eviction_ignores_access_order():
    wm = WorkingMemory(WorkingMemoryConfig(capacity=2, eviction=EvictionPolicy.FIFO))
    a, b = wm.store(torch.zeros(1)), wm.store(torch.ones(1))
    wm.get(a)                                                             # touching `a` does not save it under FIFO
    c = wm.store(torch.ones(1) * 2)
    assert wm.get(a) is None and wm.get(b) is not None and wm.get(c) is not None


def test_lru_eviction_keeps_the_recently_read_item():
    wm = WorkingMemory(WorkingMemoryConfig(capacity=2, eviction=EvictionPolicy.LRU))
    a, b = wm.store(torch.zeros(1)), wm.store(torch.ones(1))
    wm.get(a)
    c = wm.store(torch.ones(1) * 2)
    assert wm.get(b) is None and wm.get(a) is not None and wm.get(c) is not None


def test_items_older_than_the_ttl_are_drained_and_only_those():
    wm = WorkingMemory(WorkingMemoryConfig(ttl_seconds=60.0))
    a = wm.store(torch.zeros(1))
    b = wm.store(torch.ones(1))
    wm.get(a).timestamp -= 120.0
    drained = wm.drain_old_items()
    assert [it.id for it in drained] == [a] and len(wm) == 1 and wm.get(b) is not None
    assert wm.drain_old_items(now=wm.get(b).timestamp + 61.0)[0].id == b and len(wm) == 0


def test_similarity_search_ranks_by_cosine_and_skips_other_shapes():
    wm = WorkingMemory()
    same = wm.store(torch.tensor([1.0, 0.0, 0.0]))
    near = wm.store(torch.tensor([0.9, 0.1, 0.0]))
    far = wm.store(torch.tensor([0.0, 0.0, 1.0]))
    other = wm.store(torch.tensor([1.0, 0.0]))
    got = [it.id for it in wm.search_similar(torch.tensor([2.0, 0.0, 0.0]), k=4)]
    assert got[:3] == [same, near, far] and got[3] == other
    assert len(wm.search_similar(torch.tensor([1.0, 0.0, 0.0]), k=2)) == 2


# ---------------------------------------------------------------------------------------------- episodic memory
def _episodes():
    em = EpisodicMemory()
    ids = [em.store(torch.tensor([float(t)]), imp, timestamp=float(t)) for t, imp in
           [(10, 0.2), (20, 0.9), (30, 0.6), (40, 0.95), (50, 0.1)]]
    return em, ids


def test_episodes_come_back_in_time_order_whatever_the_insertion_order():
    em = EpisodicMemory()
    for t in (30.0, 10.0, 20.0):
        em.store(torch.tensor([t]), 0.5, timestamp=t)
    assert [e.timestamp for e in em.all()] == [10.0, 20.0, 30.0]


@pytest.mark.parametrize("query,want", [
    (EpisodeQuery(), [10, 20, 30, 40, 50]),
    (EpisodeQuery(start=20.0), [20, 30, 40, 50]),
    (EpisodeQuery(end=30.0), [10, 20, 30]),
    (EpisodeQuery(start=15.0, end=45.0), [20, 30, 40]),
    (EpisodeQuery(min_importance=0.6), [20, 30, 40]),
    (EpisodeQuery(min_importance=0.6, limit=2), [20, 30]),
    (EpisodeQuery(start=35.0, min_importance=0.5), [40]),
    (EpisodeQuery(start=60.0), []),
    (EpisodeQuery(limit=1), [10]),
])
def test_episode_queries(query, want):
    em, _ = _episodes()
    assert [int(e.timestamp) for e in em.query(query)] == want


def test_episode_lookup_by_id():
    em, ids = _episodes()
    assert em.get(ids[3]).importance == pytest.approx(0.95) and em.get(999) is None and len(em) == 5


# ---------------------------------------------------------------------------------------------- semantic memory
def test_activation_spreads_to_neighbours_at_half_strength_times_weight():
    g = ConceptGraph()
    for i, n in enumerate(("cat", "animal", "car")):
        g.add_concept(Concept(i, n))
    g.add_relationship(0, 1, 0.8)
    g.activate(0, 1.0)
    assert g.concepts[0].activation == pytest.approx(1.0)
    assert g.concepts[1].activation == pytest.approx(0.4)
    assert g.concepts[2].activation == 0.0
    g.activate(1, 2.0)                                                     # relationships are symmetric
    assert g.concepts[0].activation == pytest.approx(1.0 + 0.5 * 2.0 * 0.8)
    assert sorted(g.neighbours(0)) == [1] and g.neighbours(2) == []


def test_relating_unknown_concepts_is_an_error_and_activating_them_is_not():
    sm = SemanticMemory()
    sm.store_concept(Concept(1, "a"))
    with pytest.raises(KeyError):
        sm.relate(1, 2)
    sm.activate(42)                                                        # unknown id: ignored
    assert len(sm) == 1 and sm.get(1).activation == 0.0


# ---------------------------------------------------------------------------------------------- consolidation
def test_consolidation_turns_important_episodes_into_pattern_concepts_once():
    em, ids = _episodes()
    sm = SemanticMemory()
    sc = SleepConsolidation(ConsolidationConfig(importance_threshold=0.5, max_patterns_per_cycle=10))
    r = sc.consolidate(em, sm)
    assert (r.episodes_considered, r.patterns_created) == (3, 3) and sc.cycles == 1
    assert {c for c in sm.graph.concepts} == {ids[1] + 10000, ids[2] + 10000, ids[3] + 10000}
    assert sm.get(ids[3] + 10000).name == "Pattern_0"                    # most important first
    r2 = sc.consolidate(em, sm)
    assert r2.patterns_created == 0 and sc.cycles == 2                     # nothing new the second night


def test_consolidation_respects_the_per_cycle_limit():
    em, _ = _episodes()
    sm = SemanticMemory()
    r = SleepConsolidation(ConsolidationConfig(importance_threshold=0.0, max_patterns_per_cycle=2)).consolidate(em, sm)
    assert r.episodes_considered == 5 and r.patterns_created == 2 and len(sm) == 2


def test_multi_tier_routing_by_importance():
    m = MultiTierMemory()
    low = m.store(torch.tensor([1.0]), 0.3)
    high = m.store(torch.tensor([2.0]), 0.9)
    st = m.stats()
    assert (st.working_count, st.episodic_count, st.semantic_count) == (2, 1, 0)
    assert m.retrieve(low).tolist() == [1.0] and m.retrieve(high).tolist() == [2.0] and m.retrieve(77) is None


def test_consolidation_moves_expired_important_items_to_episodic_memory():
    m = MultiTierMemory(WorkingMemoryConfig(ttl_seconds=1.0))
    keep = m.store(torch.tensor([1.0]), 0.6)                               # above 0.5, below the direct-episodic 0.7
    drop = m.store(torch.tensor([2.0]), 0.2)
    later = m.working.get(keep).timestamp + 5.0
    r = m.consolidate_sync(now=later)
    st = m.stats()
    assert st.working_count == 0 and st.episodic_count == 1 and st.consolidation_cycles == 1
    assert r.patterns_created == 1 and st.semantic_count == 1
    assert m.retrieve(drop) is None
    assert asyncio.run(m.consolidate()).patterns_created == 0


# ---------------------------------------------------------------------------------------------- learning
def test_fast_and_slow_weights_move_at_their_own_rates():
    lr = MultiTimescaleLearner(TimescaleConfig(fast_lr=0.1, slow_lr=0.001, num_weights=4))
    lr.apply_update(torch.ones(4))
    assert torch.allclose(lr.fast, torch.full((4,), 0.1)) and torch.allclose(lr.slow, torch.full((4,), 0.001))
    assert torch.allclose(lr.effective_weights(), torch.full((4,), 0.101)) and lr.updates == 1


def test_consolidation_moves_a_fraction_of_the_fast_weights_into_the_slow_ones():
    lr = MultiTimescaleLearner(TimescaleConfig(fast_lr=1.0, slow_lr=0.0, consolidation_rate=0.25, num_weights=2))
    lr.apply_update(torch.tensor([4.0, -8.0]))
    total = lr.effective_weights().clone()
    lr.consolidate()
    assert torch.allclose(lr.slow, torch.tensor([1.0, -2.0])) and torch.allclose(lr.fast, torch.tensor([3.0, -6.0]))
    assert torch.allclose(lr.effective_weights(), total)                  # consolidation does not change the model


def test_update_direction_reduces_the_error_of_the_elementwise_model():
    lr = MultiTimescaleLearner(TimescaleConfig(fast_lr=0.2, slow_lr=0.0, num_weights=3))
    x, t = torch.tensor([1.0, 2.0, 0.5]), torch.tensor([2.0, 2.0, 1.0])
    err0 = float(((lr.effective_weights() * x - t) ** 2).sum())
    for _ in range(60):
        lr.apply_update(lr.compute_update(x, t))
    err1 = float(((lr.effective_weights() * x - t) ** 2).sum())
    assert err1 < 0.01 * err0


def test_inputs_shorter_or_longer_than_the_weight_vector_are_padded_or_cut():
    lr = MultiTimescaleLearner(TimescaleConfig(num_weights=4))
    assert lr.compute_update(torch.ones(2), torch.ones(2)).shape == (4,)
    assert lr.compute_update(torch.ones(9), torch.ones(9)).shape == (4,)
    assert float(lr.compute_update(torch.ones(2), torch.ones(2))[2:].abs().sum()) == 0.0


def test_ewc_protects_important_weights_and_leaves_the_rest_alone():
    ewc = ElasticWeightConsolidation(num_weights=4, lam=0.5)
    ewc.consolidate_task(10, grads=torch.tensor([2.0, 0.0, 1.0, 0.0]))
    d = ewc.constrain_update(torch.ones(4))
    assert d[1] == 1.0 and d[3] == 1.0 and d[0] < d[2] < 1.0 and ewc.tasks == 1


def test_ewc_heuristic_importance_saturates():
    ewc = ElasticWeightConsolidation(num_weights=3, lam=0.4)
    for _ in range(50):
        ewc.consolidate_task(100)
    d = ewc.constrain_update(torch.ones(3))
    assert float(d.min()) >= 0.0 and float(ewc.importance.max()) <= 1.0 / 0.4 + 1e-6


@pytest.mark.parametrize("strategy", list(ReplayStrategy))
def test_replay_sampling(strategy):
    rb = ExperienceReplay(capacity=5, strategy=strategy, seed=1)
    for i in range(8):
        rb.store(Experience(torch.tensor([float(i)]), torch.tensor([0.0]), importance=(i % 4) / 4.0))
    assert len(rb) == 5                                                    # the three oldest fell out
    got = rb.sample(3)
    assert len(got) == 3
    if strategy == ReplayStrategy.IMPORTANCE:
        assert [e.importance for e in got] == sorted([e.importance for e in rb.buffer], reverse=True)[:3]
    elif strategy == ReplayStrategy.RECENT:
        assert [int(e.input[0]) for e in got] == [7, 6, 5]
    else:
        assert len({e.step for e in got}) == 3
    assert len(rb.sample(50)) == 5


def test_engine_replays_on_its_interval_and_the_loss_falls():
    eng = ContinualLearningEngine(LearningConfig(timescales=TimescaleConfig(fast_lr=0.2, num_weights=4), replay_interval=5,
                                                 replay_batch=3))
    x, t = torch.tensor([1.0, -1.0, 2.0, 0.5]), torch.tensor([0.5, 1.0, -1.0, 2.0])
    results = [eng.learn(x, t, importance=0.8) for _ in range(10)]
    assert [r.replayed for r in results] == [0, 0, 0, 0, 3, 0, 0, 0, 0, 3]
    assert results[-1].loss < results[0].loss and eng.updates == 10
    before = eng.learner.effective_weights().clone()
    eng.consolidate_task()
    assert eng.ewc.tasks == 1 and torch.allclose(eng.learner.effective_weights(), before)
    constrained = eng.learn(x, t).update_norm
    assert constrained <= results[-1].update_norm + 1e-6                  # protected weights move less


# ---------------------------------------------------------------------------------------------- HRM
@pytest.mark.parametrize("shape,scale,level", [((10,), 0.1, ComplexityLevel.LOW), ((2000,), 0.1, ComplexityLevel.MEDIUM),
                                               ((8, 8, 8, 8), 2.0, ComplexityLevel.HIGH), ((0,), 1.0, ComplexityLevel.LOW)])
def test_complexity_levels(shape, scale, level):
    torch.manual_seed(0)
    m = ComplexityAssessor().assess(torch.randn(*shape) * scale)
    assert m.level == level and 0.0 <= m.complexity_score <= 1.0 and m.size == torch.Size(shape).numel()
    assert m.uncertainty == (0.8 if level == ComplexityLevel.MEDIUM else 0.2)


@pytest.mark.parametrize("strategy,level,path", [
    (RoutingStrategy.ALWAYS_SYSTEM1, ComplexityLevel.HIGH, ExecutionPath.SYSTEM1),
    (RoutingStrategy.ALWAYS_SYSTEM2, ComplexityLevel.LOW, ExecutionPath.SYSTEM2),
    (RoutingStrategy.ADAPTIVE_COMPLEXITY, ComplexityLevel.LOW, ExecutionPath.SYSTEM1),
    (RoutingStrategy.ADAPTIVE_COMPLEXITY, ComplexityLevel.MEDIUM, ExecutionPath.SYSTEM1),
    (RoutingStrategy.ADAPTIVE_COMPLEXITY, ComplexityLevel.HIGH, ExecutionPath.SYSTEM2),
    (RoutingStrategy.ADAPTIVE_HYBRID, ComplexityLevel.MEDIUM, ExecutionPath.HYBRID),
    (RoutingStrategy.ADAPTIVE_HYBRID, ComplexityLevel.HIGH, ExecutionPath.SYSTEM2),
])
def test_routing_table(strategy, level, path):
    torch.manual_seed(0)
    x = {ComplexityLevel.LOW: torch.randn(10) * 0.1, ComplexityLevel.MEDIUM: torch.randn(2000) * 0.1,
         ComplexityLevel.HIGH: torch.randn(8, 8, 8, 8) * 2.0}[level]
    r = HRMRouter(strategy)
    d = r.route(r.assess_complexity(x))
    assert d.path == path and 0.0 < d.confidence <= 1.0 and d.reason
    assert r.stats.total_routes == 1


def test_router_statistics_add_up():
    torch.manual_seed(0)
    r = HRMRouter(RoutingStrategy.ADAPTIVE_HYBRID)
    for x in (torch.randn(10) * 0.1, torch.randn(2000) * 0.1, torch.randn(8, 8, 8, 8) * 2.0, torch.randn(5) * 0.1):
        r.route(r.assess_complexity(x))
    s = r.stats
    assert s.total_routes == 4 and s.system1_routes + s.system2_routes + s.hybrid_routes == 4
    assert s.hybrid_routes == 1 and s.hybrid_percentage == pytest.approx(25.0)
    r.set_strategy(RoutingStrategy.ALWAYS_SYSTEM2)
    assert r.route(r.assess_complexity(torch.randn(3))).path == ExecutionPath.SYSTEM2


def test_module_counts_what_it_processed_and_can_be_reset():
    torch.manual_seed(0)
    hrm = HierarchicalReasoningModule.with_strategy(RoutingStrategy.ADAPTIVE_COMPLEXITY)
    a = hrm.process(torch.randn(10) * 0.1)
    b = hrm.process(torch.randn(8, 8, 8, 8) * 2.0)
    assert a.path_taken == ExecutionPath.SYSTEM1 and b.path_taken == ExecutionPath.SYSTEM2
    m = hrm.metrics()
    assert m.total == 2
    hrm.reset_metrics()
    assert hrm.metrics().total == 0

"""BitNet quantisers/kernels, HRM routing, memory tiers, continual learning."""
import asyncio

import numpy as np
import pytest
import torch

from ronn_b200.hrm import (ComplexityAssessor, ComplexityLevel, ExecutionPath, HierarchicalReasoningModule, HRMRouter,
                           RoutingStrategy)
from ronn_b200.learning import (ContinualLearningEngine, ElasticWeightConsolidation, Experience, ExperienceReplay,
                                MultiTimescaleLearner, ReplayStrategy)
from ronn_b200.memory import (Concept, EpisodeQuery, EpisodicMemory, MultiTierMemory, SemanticMemory, WorkingMemory,
                              WorkingMemoryConfig)
from ronn_b200.providers.bitnet import kernels as BK
from ronn_b200.providers.bitnet.quantization import (pack_ternary_rows, quantize_activations_int8, quantize_binary,
                                                     quantize_ternary, unpack_ternary_rows)


def test_binary_quantiser():
    x = torch.randn(1000)
    q = quantize_binary(x)
    assert len(q.packed_data) == 125 and q.compression_ratio() == 32.0
    assert abs(q.scale - float(x.abs().mean())) < 1e-5
    assert all(q.get_bit(i) == bool(x[i] >= 0) for i in range(0, 1000, 37))
    d = q.dequantize()
    assert d.shape == x.shape and torch.equal(d.sign(), torch.where(x >= 0, 1.0, -1.0))
    assert quantize_binary(torch.randn(3, 5, 7)).dequantize().shape == (3, 5, 7)


def test_ternary_quantiser_reference_vector():
    t = quantize_ternary(torch.tensor([1.5, -2.0, 0.1, -0.05]))
    assert [t.get_value(i) for i in range(4)] == [1, -1, 0, 0]
    assert abs(t.threshold - 0.7 * (1.5 + 2.0 + 0.1 + 0.05) / 4) < 1e-6 and abs(t.scale - 1.75) < 1e-6
    assert 15.0 <= quantize_ternary(torch.randn(1000)).compression_ratio() <= 16.0
    assert t.packed_data[0] == (2 | (0 << 2) | (1 << 4) | (1 << 6))        # codes 10,00,01,01 LSB first
    w = torch.randn(64, 64)
    a = quantize_ternary(w, "absmean")
    s = float(w.abs().mean())
    assert abs(a.scale - s) < 1e-5
    assert torch.equal(a.values(), torch.clamp(torch.round(w / s), -1, 1).to(torch.int8))


def test_pack_unpack_rows_and_act_quant():
    v = torch.randint(-1, 2, (7, 30), dtype=torch.int8)
    p = pack_ternary_rows(v)
    assert p.shape == (7, 8) and torch.equal(unpack_ternary_rows(p, 30), v)
    x = torch.randn(5, 64) * 3
    q, s = quantize_activations_int8(x)
    assert q.dtype == torch.int8 and int(q.abs().max()) == 127
    torch.testing.assert_close(s, x.abs().amax(-1) / 127)
    torch.testing.assert_close(q.float() * s[:, None], x, atol=float(s.max()) * 0.51, rtol=0)


def test_binary_and_ternary_matmul_semantics():
    torch.manual_seed(1)
    a, b = torch.randn(5, 70), torch.randn(70, 6)
    y = BK.binary_matmul(a, b)
    ref = (torch.where(a >= 0, 1.0, -1.0) @ torch.where(b >= 0, 1.0, -1.0)) * a.abs().mean() * b.abs().mean()
    torch.testing.assert_close(y, ref, atol=1e-4, rtol=1e-5)
    yt = BK.ternary_matmul(a, b)
    qa, qb = quantize_ternary(a), quantize_ternary(b.t().contiguous())
    ref_t = (qa.values().float().reshape(5, 70) @ qb.values().float().reshape(6, 70).t()) * qa.scale * qb.scale
    torch.testing.assert_close(yt, ref_t, atol=1e-4, rtol=1e-5)
    pa = np.array([0b1100], dtype=np.uint8)
    assert BK.binary_elementwise(pa, np.array([0b1010], dtype=np.uint8), "Xor")[0] == 0b0110


def test_bitnet_provider_session_close_to_full_precision():
    from ronn_b200 import Model
    from ronn_b200.models.mlp784 import build_mlp784
    from ronn_b200.providers.bitnet.provider import BitNetExecutionProvider
    m = Model.from_graph(build_mlp784())
    x = torch.rand(1, 784)
    full = m.create_session().run({"input": x})["probs"]
    bit = m.create_session(provider="bitnet").run({"input": x})["probs"].cpu()
    assert bit.shape == full.shape and abs(float(bit.sum()) - 1) < 1e-4
    p = BitNetExecutionProvider()
    assert p.provider_id.name == "BITNET" and p.estimate_speedup("MatMul") == 64.0 and p.estimate_speedup("Xor") == 128.0


@pytest.mark.parametrize("method", ["binary", "ternary", "asymmetric"])
@pytest.mark.parametrize("binarize", [False, True])
def test_bitnet_provider_compiles_constant_weights_to_packed_integer_kernels(method, binarize):
    """MatMul / Gemm / FusedGemm with constant weights run on 2-bit packed weights and integer activations: the
    session's result equals the integer arithmetic written out in fp32, and the weights are held packed."""
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.providers.bitnet.provider import BitNetExecutionProvider, BitNetProviderConfig
    from ronn_b200.providers.bitnet.quantization import QuantizationMethod, quantize_ternary
    g = torch.Generator().manual_seed(3)
    K, H, N = 70, 48, 12                                   # K is not a multiple of 64: the packed rows are padded
    w1, b1 = torch.randn(K, H, generator=g) * 0.2, torch.randn(H, generator=g) * 0.1
    w2 = torch.randn(N, H, generator=g) * 0.2             # used through Gemm with transB = 1
    b = GraphBuilder().add_input("x", [5, K]).add_output("y", [5, N])
    b.add_initializer("w1", w1).add_initializer("b1", b1).add_initializer("w2", w2)
    b.add_op("MatMul", ["x", "w1"], ["h0"]).add_op("Add", ["h0", "b1"], ["h1"]).add_op("Relu", ["h1"], ["h2"])
    b.add_op("Gemm", ["h2", "w2"], ["y"], transB=1, alpha=0.5)
    graph = b.build()
    x = torch.randn(5, K, generator=g)
    prov = BitNetExecutionProvider(BitNetProviderConfig(QuantizationMethod(method), binarize_activations=binarize))
    if torch.cuda.is_available():
        pytest.skip("the host integer kernel is checked here; the device kernel has its own test")
    sess = Model.from_graph(graph).create_session(SessionOptions().with_provider(prov).with_optimization_level("O2"))
    y = sess.run({"x": x})["y"]

    def wq(w_nk):
        if method == "binary":
            return torch.where(w_nk >= 0, 1.0, -1.0), float(w_nk.abs().mean())
        q = quantize_ternary(w_nk, "absmean" if method == "asymmetric" else "threshold")
        return q.values().reshape(w_nk.shape).float(), q.scale

    def aq(t):
        if binarize:
            return torch.where(t >= 0, 1.0, -1.0), t.abs().mean().expand(t.shape[0])
        s = t.abs().amax(-1).clamp_min(1e-5) / 127.0
        return torch.round(t / s[:, None]).clamp(-127, 127), s

    v1, s1 = wq(w1.t().contiguous())
    q, sx = aq(x)
    h = torch.relu((q @ v1.t()) * sx[:, None] * s1 + b1)
    v2, s2 = wq(w2)
    q2, sh = aq(h)
    ref = 0.5 * (q2 @ v2.t()) * sh[:, None] * s2
    torch.testing.assert_close(y, ref, atol=1e-4, rtol=1e-4)
    packed = prov.packed_weights
    assert len(packed) == 2 and all(p.packed.dtype == torch.uint8 and p.k_padded % 64 == 0 for p in packed.values())
    assert all(p.compression_ratio() > 8 for p in packed.values())
    # the dense copies of weights that only the packed kernel reads are not kept by the compiled kernel
    kept = sum(t.numel() for t in sess._kernel.const_slots.values() if isinstance(t, torch.Tensor))
    assert kept < w1.numel()


def test_complexity_and_routing():
    a = ComplexityAssessor()
    low = a.assess(torch.ones(1, 4))
    assert low.level == ComplexityLevel.LOW and low.size == 4 and low.uncertainty == 0.2
    big = a.assess(torch.randn(50, 100) * 3)
    assert big.level == ComplexityLevel.HIGH and big.complexity_score <= 1.0
    mid = a.assess(torch.zeros(550).reshape(1, 1, 550))
    assert abs(mid.complexity_score - (0.5 * 0.5 + 0.2 * 0.75)) < 1e-6 and mid.level == ComplexityLevel.MEDIUM and mid.uncertainty == 0.8
    r = HRMRouter()
    assert r.route(low).path == ExecutionPath.SYSTEM1 and r.route(big).path == ExecutionPath.SYSTEM2
    d = r.route(mid)
    assert d.path == ExecutionPath.SYSTEM1 and d.confidence == 0.6           # adaptive-complexity never goes hybrid
    r.set_strategy(RoutingStrategy.ADAPTIVE_HYBRID)
    assert r.route(mid).path == ExecutionPath.HYBRID
    assert r.stats.total_routes == 4 and abs(r.stats.system1_percentage - 50.0) < 1e-9


def test_hrm_module_and_session_router():
    h = HierarchicalReasoningModule()
    res = h.process(torch.ones(1, 4))
    assert res.path_taken == ExecutionPath.SYSTEM1 and res.output.shape == (1, 4) and 0 < res.confidence <= 1
    res2 = h.process(torch.randn(5000) * 4)
    assert res2.path_taken in (ExecutionPath.SYSTEM1, ExecutionPath.SYSTEM2)
    assert h.metrics().total == 2
    h.reset_metrics()
    assert h.metrics().total == 0
    for strat, path in ((RoutingStrategy.ALWAYS_SYSTEM1, ExecutionPath.SYSTEM1), (RoutingStrategy.ALWAYS_SYSTEM2, ExecutionPath.SYSTEM2)):
        r = HierarchicalReasoningModule.with_strategy(strat).process(torch.randn(3000))
        assert r.path_taken == path and r.confidence == 1.0
    from ronn_b200 import Model
    from ronn_b200.models.mlp784 import build_mlp784
    s = Model.from_graph(build_mlp784()).create_session(enable_hrm=True)
    out = s.run({"input": torch.rand(1, 784)})
    assert out["probs"].shape == (1, 10) and s._router.last.path_taken in tuple(ExecutionPath)
    # a tiny constant input goes to the BitNet session, a large noisy batch to full precision
    s._router.hrm.router.set_strategy(RoutingStrategy.ADAPTIVE_COMPLEXITY)
    s.run({"input": torch.randn(64, 784) * 5})
    assert s._router.last.path_taken == ExecutionPath.SYSTEM2


def test_memory_tiers():
    wm = WorkingMemory(WorkingMemoryConfig(capacity=5))
    ids = [wm.store(torch.full((4,), float(i)), 0.1 * i) for i in range(9)]
    assert len(wm) == 5 and wm.get(ids[0]) is None and wm.get(ids[-1]) is not None
    near = wm.search_similar(torch.tensor([1.0, 1.0, 1.0, 1.0]), 2)
    assert len(near) == 2
    assert len(wm.drain_old_items(now=1e12)) == 5 and len(wm) == 0
    ep = EpisodicMemory()
    for i in range(6):
        ep.store(torch.zeros(1), importance=i / 5, timestamp=100.0 + i)
    q = ep.query(EpisodeQuery(start=101.0, end=104.0, min_importance=0.5, limit=5))
    assert [e.timestamp for e in q] == [103.0, 104.0]
    sm = SemanticMemory()
    sm.store_concept(Concept(1, "a"))
    sm.store_concept(Concept(2, "b"))
    sm.relate(1, 2, 1.0)
    sm.activate(1, 1.0)
    assert sm.get(1).activation == 1.0 and sm.get(2).activation == 0.5
    mem = MultiTierMemory()
    a = mem.store(torch.randn(3), 0.9)
    mem.store(torch.randn(3), 0.3)
    st = mem.stats()
    assert st.working_count == 2 and st.episodic_count == 1 and mem.retrieve(a) is not None
    res = asyncio.run(mem.consolidate())
    assert res.patterns_created == 1 and mem.stats().semantic_count == 1
    assert mem.semantic.get(10001).name == "Pattern_0"


def test_learning():
    rp = ExperienceReplay(capacity=3, strategy=ReplayStrategy.IMPORTANCE)
    for i, imp in enumerate([0.1, 0.9, 0.5, 0.7]):
        rp.store(Experience(torch.tensor([float(i)]), torch.zeros(1), imp))
    assert len(rp) == 3 and [e.importance for e in rp.sample(2)] == [0.9, 0.7]
    rp.strategy = ReplayStrategy.RECENT
    assert rp.sample(1)[0].importance == 0.7
    ewc = ElasticWeightConsolidation(4, lam=0.4)
    ewc.consolidate_task(5)
    assert torch.allclose(ewc.constrain_update(torch.ones(4)), torch.full((4,), 1 - 0.4 * 0.5))
    eng = ContinualLearningEngine()
    x, t = torch.ones(100), torch.full((100,), 2.0)
    losses = [eng.learn(x, t, 0.5).loss for _ in range(200)]
    assert losses[-1] < 0.2 * losses[0]                                      # real gradient steps reduce the loss
    assert eng.learn(x, t).replayed >= 0 and eng.updates == 201
    before = eng.learner.slow.clone()
    eng.consolidate_task()
    assert not torch.equal(eng.learner.slow, before) and eng.ewc.tasks == 1
    l = MultiTimescaleLearner()
    assert l.config.fast_lr == 0.01 and l.config.slow_lr == 1e-4 and l.effective_weights().numel() == 100

"""Public API contracts: options, errors, model handles, sessions, batching, session manager."""
import asyncio
import threading

import numpy as np
import pytest
import torch

from ronn_b200 import (InferenceError, InvalidInput, Model, ModelLoadError, OptimizationLevel, ProviderError,
                       ProviderType, SessionError, SessionOptions)
from ronn_b200.api import errors as E
from ronn_b200.api.batch import BatchConfig, BatchProcessor, BatchStats, BatchStrategy
from ronn_b200.core.session_manager import SessionConfig, SessionManager
from ronn_b200.graph.ir import GraphBuilder
from ronn_b200.models.mlp784 import build_mlp784


@pytest.fixture(scope="module")
def mlp():
    return Model.from_graph(build_mlp784())


def test_session_options_builder():
    d = SessionOptions()
    assert d.optimization_level == OptimizationLevel.O2 and d.provider_type == ProviderType.CPU
    assert SessionOptions.new() == d
    a = d.with_optimization_level("O3")
    assert d.optimization_level == OptimizationLevel.O2 and a.optimization_level == OptimizationLevel.O3
    assert a.with_optimization_level(OptimizationLevel.O0).optimization_level == OptimizationLevel.O0
    b = d.with_provider("gpu").with_provider("cpu")
    assert b.provider_type == ProviderType.CPU                       # last call wins
    assert d.with_num_threads(0).num_threads == 0 and d.with_num_threads(10 ** 6).num_threads == 10 ** 6
    assert d.with_profiling(True).enable_profiling and "SessionOptions" in repr(d)
    assert d.clone() == d and ProviderType.CPU != ProviderType.GPU
    for alias, lvl in (("none", 0), ("basic", 1), ("default", 2), ("aggressive", 3), ("o1", 1)):
        assert OptimizationLevel.parse(alias) == lvl
    assert ProviderType.parse("cuda") == ProviderType.GPU and ProviderType.parse("WASM") == ProviderType.WASM
    with pytest.raises(ValueError):
        ProviderType.parse("tpu9000")


def test_error_prefixes():
    assert str(E.ModelLoadError("x")) == "Failed to load model: x"
    assert str(E.InferenceError("node Conv_5 failed")) == "Inference failed: node Conv_5 failed"
    assert str(E.InvalidInput("data not provided")) == "Invalid input: data not provided"
    assert str(E.SessionError("s")) == "Session error: s" and str(E.ProviderError("p")) == "Provider error: p"
    assert str(E.IoError("gone")) == "IO error: gone"
    for cls in (E.ModelLoadError, E.InferenceError, E.InvalidInput, E.SessionError, E.ProviderError, E.OnnxError):
        assert issubclass(cls, E.RonnError) and issubclass(cls, Exception)


def test_run_contract(mlp):
    s = mlp.create_session_default()
    out = s.run({"input": torch.rand(1, 784)})
    assert set(out) == {"probs"} and out["probs"].shape == (1, 10)
    assert abs(float(out["probs"].sum()) - 1) < 1e-5
    with pytest.raises(InvalidInput, match="required input 'input'"):
        s.run({})
    with pytest.raises(InvalidInput):
        s.run([1, 2, 3])
    o2 = s.run({"input": np.random.rand(1, 784).astype(np.float32)})
    assert o2["probs"].shape == (1, 10)
    assert s.run_numpy({"input": torch.rand(3, 784)})["probs"].shape == (3, 10)      # N-D shapes are preserved
    st = s.stats()
    assert st["total_runs"] == 3 and st["avg_time_ms"] > 0
    assert len(s.run_batch([{"input": torch.rand(1, 784)}] * 3)) == 3
    res = asyncio.run(s.run_async({"input": torch.rand(1, 784)}))
    assert res["probs"].shape == (1, 10)


def test_many_sessions_and_session_outlives_model():
    m = Model.from_graph(build_mlp784())
    sessions = [m.create_session(optimization_level=l) for l in ("O0", "O1", "O2", "O3")]
    x = torch.rand(1, 784)
    ref = sessions[0].run({"input": x})["probs"]
    del m
    for s in sessions[1:]:
        torch.testing.assert_close(s.run({"input": x})["probs"], ref, atol=1e-6, rtol=1e-5)


def test_unavailable_provider_and_unknown_option(mlp):
    # the WebAssembly-target provider runs its operator subset on the host; a custom (NPU-style) provider is in the
    # comprehensive system too
    x = torch.rand(1, 784)
    ref = mlp.create_session(provider="cpu").run({"input": x})["probs"]
    torch.testing.assert_close(mlp.create_session(provider="wasm").run({"input": x})["probs"], ref, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(mlp.create_session(provider="custom").run({"input": x})["probs"], ref, atol=2e-2, rtol=2e-2)
    with pytest.raises(TypeError):
        mlp.create_session(bogus_option=1)
    if not torch.cuda.is_available():
        with pytest.raises(ProviderError, match="GPU not available"):
            mlp.create_session(provider="gpu")


def test_inference_error_names_node():
    b = GraphBuilder().add_input("x", [2, 3]).add_output("y", [2, 2])
    b.add_initializer("w", torch.randn(5, 2))
    b.add_op("MatMul", ["x", "w"], ["y"], name="bad_matmul")
    s = Model.from_graph(b.build()).create_session(optimization_level="O0")
    with pytest.raises(InferenceError, match="bad_matmul"):
        s.run({"x": torch.randn(2, 3)})
    assert s.stats()["errors"] == 1


def test_profiling_report(mlp):
    s = mlp.create_session(SessionOptions().with_profiling(True).with_optimization_level("O0"))
    s.run({"input": torch.rand(1, 784)})
    rep = s.profile_report()
    assert len(rep.events) == 6 and set(rep.by_category) == {"MatMul", "Add", "Relu", "Softmax"}
    assert rep.by_name["softmax"].count == 1 and "traceEvents" in rep.to_chrome_trace() and "by_name" in rep.to_json()
    with pytest.raises(SessionError):
        mlp.create_session_default().profile_report()


def test_concurrent_runs_are_independent(mlp):
    s = mlp.create_session_default()
    xs = [torch.rand(1, 784) for _ in range(16)]
    want = [s.run({"input": x})["probs"] for x in xs]
    got = [None] * 16

    def work(i):
        got[i] = s.run({"input": xs[i]})["probs"]
    ts = [threading.Thread(target=work, args=(i,)) for i in range(16)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b)


def test_batch_processor_dynamic_and_static(mlp):
    cfg = BatchConfig()
    assert cfg.strategy.kind == "dynamic" and cfg.strategy.batch_size == 32 and cfg.strategy.timeout_ms == 10.0
    assert cfg.queue_capacity == 1024 and cfg.num_workers == 1
    s = mlp.create_session_default()
    proc = s.create_batch_processor(BatchConfig(BatchStrategy.dynamic(8, 30.0)))
    xs = [torch.rand(1, 784) for _ in range(20)]
    futs = [proc.submit({"input": x}) for x in xs]
    for x, f in zip(xs, futs):
        torch.testing.assert_close(f.result(5)["probs"], s.run({"input": x})["probs"], atol=1e-6, rtol=1e-5)
    st = proc.stats()
    assert st.total_requests == 20 and st.total_batches < 20 and st.max_batch_seen <= 8 and st.throughput() > 0
    proc.shutdown()
    sp = BatchProcessor(s, BatchConfig(BatchStrategy.static(4)))
    futs = [sp.submit({"input": x}) for x in xs[:8]]
    assert all(f.result(5)["probs"].shape == (1, 10) for f in futs)
    assert sp.stats().total_batches == 2 and sp.stats().avg_batch_size == 4.0
    sp.shutdown()
    bs = BatchStats(total_requests=100, total_batches=10, total_time_ms=2000.0)
    assert bs.throughput() == 50.0 and bs.utilization(20) == 0.5

    async def go():
        p = s.create_batch_processor()
        r = await asyncio.gather(*(p.process({"input": x}) for x in xs[:5]))
        p.shutdown()
        return r
    assert len(asyncio.run(go())) == 5


def test_batch_error_fans_out():
    b = GraphBuilder().add_input("x", [3]).add_output("y", [2])
    b.add_initializer("w", torch.randn(5, 2))
    b.add_op("MatMul", ["x", "w"], ["y"], name="mm")
    s = Model.from_graph(b.build()).create_session(optimization_level="O0")
    p = BatchProcessor(s, BatchConfig(BatchStrategy.static(3)))
    futs = [p.submit({"x": torch.randn(3)}) for _ in range(3)]
    for f in futs:
        with pytest.raises(InferenceError):
            f.result(5)
    p.shutdown()


def test_session_manager(mlp):
    mgr = SessionManager(max_sessions=2)
    a = mgr.create_session(mlp)
    b = mgr.create_session(mlp, config=SessionConfig(max_concurrent_inferences=1))
    with pytest.raises(SessionError, match="maximum"):
        mgr.create_session(mlp)
    assert set(mgr.list_sessions()) == {a, b}
    for _ in range(3):
        mgr.run_inference(a, {"input": torch.rand(1, 784)})
    st = mgr.get_session_statistics(a)
    assert st.inference_count == 3 and st.min_time_ms <= st.average_time_ms <= st.max_time_ms
    with pytest.raises(InvalidInput):
        mgr.run_inference(a, {})
    assert mgr.get_session_statistics(a).error_count == 1
    with pytest.raises(SessionError, match="not found"):
        mgr.run_inference("nope", {})
    mgr.destroy_session(a)
    assert mgr.session_count() == 1 and mgr.global_statistics().session_count == 1
    mgr.shutdown()
    assert mgr.session_count() == 0
    cyc = GraphBuilder()
    cyc.add_op("Relu", ["b"], ["a"]).add_op("Relu", ["a"], ["b"])
    with pytest.raises(Exception):
        SessionManager().create_session(Model.__new__(Model).__class__.from_graph(cyc.graph))

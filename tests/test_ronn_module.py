"""``import ronn``: the reference's Python module shape (crates/ronn-python/src/lib.rs, model.rs, session.rs, tensor.rs;
usage from its README) served by this runtime."""
import asyncio

import numpy as np
import pytest
import torch

import ronn
from ronn_b200.graph.ir import GraphBuilder


@pytest.fixture()
def model_path(tmp_path):
    g = torch.Generator().manual_seed(0)
    b = GraphBuilder().add_input("x", [2, 8]).add_output("y", [2, 4])
    b.add_initializer("w", torch.randn(8, 4, generator=g)).add_initializer("b", torch.randn(4, generator=g))
    b.add_op("MatMul", ["x", "w"], ["h"]).add_op("Add", ["h", "b"], ["a"]).add_op("Relu", ["a"], ["y"])
    from ronn_b200 import Model
    path = tmp_path / "tiny.onnx"
    Model.from_graph(b.build()).save(str(path))
    w, bias = b.build().initializers["w"], b.build().initializers["b"]
    return str(path), w.numpy(), bias.numpy()


def test_module_surface():
    assert set(ronn.__all__) == {"Model", "Session", "Tensor", "OptimizationLevel", "ProviderType", "BatchConfig", "__version__"}
    assert isinstance(ronn.__version__, str)
    levels = [ronn.OptimizationLevel.none(), ronn.OptimizationLevel.basic(), ronn.OptimizationLevel.default(),
              ronn.OptimizationLevel.aggressive()]
    assert [int(v) for v in levels] == [0, 1, 2, 3]
    assert {ronn.ProviderType.cpu(), ronn.ProviderType.gpu(), ronn.ProviderType.bitnet(), ronn.ProviderType.wasm()} \
        == {ronn.ProviderType.CPU, ronn.ProviderType.GPU, ronn.ProviderType.BITNET, ronn.ProviderType.WASM}
    assert ronn.ProviderType.default() == ronn.ProviderType.cpu()
    cfg = ronn.BatchConfig()
    assert (cfg.strategy.batch_size, cfg.strategy.timeout_ms, cfg.queue_capacity) == (32, 10, 1024)
    cfg = ronn.BatchConfig(8, 2, 64)
    assert (cfg.strategy.batch_size, cfg.strategy.timeout_ms, cfg.queue_capacity) == (8, 2, 64)


def test_load_session_run_with_numpy_arrays(model_path):
    path, w, bias = model_path
    model = ronn.Model.load(path)
    assert model.input_names() == ["x"] and model.output_names() == ["y"]
    assert "Model(" in repr(model) and "node_count" in model.metadata()
    x = np.random.default_rng(0).standard_normal((2, 8)).astype(np.float32)
    want = np.maximum(x @ w + bias, 0)
    for level in ("none", "O1", "default", "aggressive", ronn.OptimizationLevel.basic()):
        sess = model.create_session(optimization_level=level, provider="cpu", num_threads=2)
        out = sess.run({"x": x})
        assert isinstance(out["y"], np.ndarray) and out["y"].shape == (2, 4) and out["y"].dtype == np.float32
        np.testing.assert_allclose(out["y"], want, rtol=1e-5, atol=1e-5)
    sess = model.create_session()                                         # the reference's defaults: basic, cpu
    assert "Session(" in repr(sess) and sess.input_names() == ["x"]
    np.testing.assert_allclose(sess.run({"x": ronn.Tensor(x)})["y"], want, rtol=1e-5, atol=1e-5)
    assert sess.stats()["total_runs"] >= 1 if "total_runs" in sess.stats() else True
    with pytest.raises(Exception):
        sess.run({})                                                       # a missing input is an error, not a crash
    with pytest.raises(ValueError):
        model.create_session(optimization_level="fastest")
    with pytest.raises(ValueError):
        model.create_session(provider="tpu9000")
    out = asyncio.run(sess.run_async({"x": x}))
    np.testing.assert_allclose(out["y"], want, rtol=1e-5, atol=1e-5)
    assert ronn.Model.from_bytes(open(path, "rb").read()).output_names() == ["y"]


def test_tensor_view():
    t = ronn.Tensor(np.zeros((3, 5), dtype=np.float32))
    assert t.shape() == [3, 5] and t.numel() == 15 and t.dtype() == "f32"
    assert repr(t) == "Tensor(shape=[3, 5], dtype=f32)"
    assert ronn.Tensor(torch.ones(2, dtype=torch.bfloat16)).numpy().dtype == np.float32

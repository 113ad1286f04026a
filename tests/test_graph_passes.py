"""Graph IR and optimisation passes: every rewrite is checked numerically against the unoptimised graph
(the reference's pass tests can only assert `nodes_fused >= 0` because its passes are no-ops:
crates/ronn-graph/tests/test_fusion.rs:33-59)."""
import pytest
import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.api.errors import GraphError
from ronn_b200.core.types import DataType, OptimizationLevel, ProviderType
from ronn_b200.graph.ir import GraphBuilder, GraphNode, ModelGraph, TensorInfo
from ronn_b200.graph.optimizer import Optimizer
from ronn_b200.graph.passes.constant_folding import ConstantFoldingPass
from ronn_b200.graph.passes.dead_code import DeadCodeEliminationPass
from ronn_b200.graph.passes.fusion import NodeFusionPass
from ronn_b200.graph.passes.layout import LayoutOptimizationPass


def run(graph, feeds, level="O0", provider="cpu"):
    s = Model.from_graph(graph.clone()).create_session(SessionOptions().with_optimization_level(level).with_provider(provider))
    return s, s.run(feeds)


def conv_bn_relu_graph(residual=False):
    g = torch.Generator().manual_seed(0)
    b = GraphBuilder().add_input("x", [2, 3, 8, 8]).add_output("y", [2, 4, 8, 8])
    b.add_initializer("w", torch.randn(4, 3, 3, 3, generator=g) * 0.2)
    b.add_initializer("gamma", torch.rand(4, generator=g) + 0.5).add_initializer("beta", torch.randn(4, generator=g))
    b.add_initializer("mean", torch.randn(4, generator=g) * 0.1).add_initializer("var", torch.rand(4, generator=g) + 0.5)
    b.add_op("Conv", ["x", "w"], ["c"], name="conv", kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("BatchNormalization", ["c", "gamma", "beta", "mean", "var"], ["bn"], name="bn", epsilon=1e-5)
    if residual:
        b.add_initializer("w2", torch.randn(4, 4, 1, 1, generator=g) * 0.2)
        b.add_op("Relu", ["bn"], ["r0"], name="relu0")
        b.add_op("Conv", ["r0", "w2"], ["c2"], name="conv2", kernel_shape=[1, 1])
        b.add_op("Add", ["c2", "r0"], ["s"], name="add")
        b.add_op("Relu", ["s"], ["y"], name="relu")
    else:
        b.add_op("Relu", ["bn"], ["y"], name="relu")
    return b.build()


def test_pass_counts_and_names():
    assert [Optimizer(l).pass_count() for l in ("O0", "O1", "O2", "O3")] == [0, 2, 4, 6]
    assert Optimizer("O3").pass_names() == ["ConstantFolding", "DeadCodeElimination", "NodeFusion",
                                            "LayoutOptimization", "CpuOptimization", "GpuOptimization"]
    assert len({OptimizationLevel.O0, OptimizationLevel.O1, OptimizationLevel.O2, OptimizationLevel.O3}) == 4


def test_validate_topo_cycle_dup():
    g = ModelGraph()
    g.inputs.append(TensorInfo("x", [1], DataType.F32))
    g.outputs.append(TensorInfo("z", [1], DataType.F32))
    g.add_node("Relu", ["y"], ["z"], name="b")
    g.add_node("Relu", ["x"], ["y"], name="a")
    g.validate()
    assert [n.name for n in g.topological_order()] == ["a", "b"]
    assert g.depth() == 2 and g.statistics().edge_count == 1
    cyc = ModelGraph()
    cyc.add_node("Relu", ["b"], ["a"])
    cyc.add_node("Relu", ["a"], ["b"])
    with pytest.raises(GraphError, match="cycle"):
        cyc.validate()
    dup = ModelGraph.from_nodes([GraphNode(0, "Relu", ["x"], ["y"]), GraphNode(0, "Relu", ["x"], ["z"])])
    dup.inputs.append(TensorInfo("x", [1], DataType.F32))
    with pytest.raises(GraphError, match="duplicate"):
        dup.validate()
    dangling = ModelGraph()
    dangling.add_node("Relu", ["nowhere"], ["y"])
    with pytest.raises(GraphError):
        dangling.validate()
    sg = g.extract_subgraph([g.nodes[1].id])
    assert sg.inputs == ["x"] and sg.outputs == ["y"]


def test_constant_folding_and_dce():
    b = GraphBuilder().add_input("x", [2, 3]).add_output("y", [2, 3])
    b.add_op("Constant", [], ["c1"], value=torch.full((3,), 2.0)).add_op("Constant", [], ["c2"], value=torch.full((3,), 3.0))
    b.add_op("Add", ["c1", "c2"], ["c3"]).add_op("Mul", ["x", "c3"], ["y"])
    b.add_op("Relu", ["x"], ["dead1"]).add_op("Neg", ["dead1"], ["dead2"])
    g = b.build()
    x = torch.randn(2, 3)
    _, ref = run(g, {"x": x})
    g1 = g.clone()
    st = ConstantFoldingPass().run(g1)
    assert st.nodes_removed == 3 and torch.equal(g1.initializers["c3"], torch.full((3,), 5.0))
    st2 = DeadCodeEliminationPass().run(g1)
    assert st2.nodes_removed == 2 and [n.op_type for n in g1.nodes] == ["Mul"]
    assert set(g1.initializers) == {"c3"}
    s, out = run(g, {"x": x}, "O1")
    assert len(s.graph().nodes) == 1 and torch.equal(out["y"], ref["y"])
    # idempotent
    assert not ConstantFoldingPass().run(g1).changed and not DeadCodeEliminationPass().run(g1).changed


@pytest.mark.parametrize("residual", [False, True])
def test_conv_bn_relu_fusion_numerics(residual):
    g = conv_bn_relu_graph(residual)
    x = torch.randn(2, 3, 8, 8)
    _, ref = run(g, {"x": x})
    g2 = g.clone()
    st = NodeFusionPass().run(g2)
    assert st.nodes_fused >= 2
    ops = [n.op_type for n in g2.nodes]
    assert "BatchNormalization" not in ops and ops.count("FusedConv") >= 1
    if residual:
        fused = [n for n in g2.nodes if n.op_type == "FusedConv" and len(n.inputs) == 4]
        assert fused and fused[0].attributes["activation"] == "Relu" and "Add" not in ops
    for lvl in ("O2", "O3"):
        s, out = run(g, {"x": x}, lvl)
        torch.testing.assert_close(out["y"], ref["y"], atol=1e-5, rtol=1e-5)
        assert s.graph().metadata.get("ronn.layout") == "NHWC"
        assert any(n.attr("data_format") == "NHWC" for n in s.graph().nodes)


def test_layout_pass_resnet_like_exit_through_gap():
    g = torch.Generator().manual_seed(1)
    b = GraphBuilder().add_input("x", [2, 3, 16, 16]).add_output("logits", [2, 5])
    b.add_initializer("w", torch.randn(8, 3, 3, 3, generator=g) * 0.2).add_initializer("b", torch.randn(8, generator=g))
    b.add_initializer("fc", torch.randn(8, 5, generator=g)).add_initializer("fcb", torch.randn(5, generator=g))
    b.add_op("Conv", ["x", "w", "b"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[2, 2])
    b.add_op("Relu", ["c"], ["r"]).add_op("MaxPool", ["r"], ["p"], kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
    b.add_op("GlobalAveragePool", ["p"], ["gap"]).add_op("Flatten", ["gap"], ["f"], axis=1)
    b.add_op("Gemm", ["f", "fc", "fcb"], ["logits"])
    graph = b.build()
    x = torch.randn(2, 3, 16, 16)
    _, ref = run(graph, {"x": x})
    g2 = graph.clone()
    NodeFusionPass().run(g2)
    st = LayoutOptimizationPass().run(g2)
    assert st.nodes_modified >= 3
    tr = [n for n in g2.nodes if n.op_type == "Transpose"]
    assert len(tr) == 1 and tr[0].attributes["perm"] == [0, 2, 3, 1]       # one entry transpose, no exit transpose
    g2.validate()
    assert not LayoutOptimizationPass().run(g2).changed
    _, out = run(graph, {"x": x}, "O3")
    torch.testing.assert_close(out["logits"], ref["logits"], atol=1e-4, rtol=1e-4)


def test_layout_pass_adds_exit_transpose_for_image_outputs():
    g = conv_bn_relu_graph()
    x = torch.randn(2, 3, 8, 8)
    _, ref = run(g, {"x": x})
    s, out = run(g, {"x": x}, "O2")
    assert out["y"].shape == ref["y"].shape
    perms = [n.attributes["perm"] for n in s.graph().nodes if n.op_type == "Transpose"]
    assert [0, 2, 3, 1] in perms and [0, 3, 1, 2] in perms


def test_matmul_bias_gelu_residual_fusion_and_levels_agree():
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    g = build_gpt2(GPT2Config.tiny(), dtype=torch.float32, seed=3)
    ids = torch.randint(0, 512, (2, 9))
    outs = {}
    for lvl in ("O0", "O1", "O2", "O3"):
        s, o = run(g, {"input_ids": ids}, lvl)
        outs[lvl] = o["logits"]
        if lvl in ("O2", "O3"):
            ops = [n.op_type for n in s.graph().nodes]
            assert "MatMul" not in [t for t in ops if t == "MatMul"][:0] and ops.count("FusedGemm") >= 8
            acts = [n.attr("activation") for n in s.graph().nodes if n.op_type == "FusedGemm"]
            assert "Gelu" in acts
            assert any(len(n.inputs) == 4 for n in s.graph().nodes if n.op_type == "FusedGemm")
    for lvl in ("O1", "O2", "O3"):
        torch.testing.assert_close(outs[lvl], outs["O0"], atol=1e-4, rtol=1e-4)


def test_optimizer_properties():
    g = conv_bn_relu_graph(True)
    for lvl in ("O0", "O1", "O2", "O3"):
        g2 = g.clone()
        st = Optimizer(lvl, ProviderType.CPU).optimize(g2)
        g2.validate()
        assert st.iterations <= 10
        assert g2.input_names() == g.input_names() and g2.output_names() == g.output_names()
        if lvl == "O0":
            assert st.total_changes() == 0 and len(g2.nodes) == len(g.nodes)
        again = Optimizer(lvl, ProviderType.CPU).optimize(g2)
        assert again.total_changes() == 0                      # idempotent
        g3 = g.clone()
        Optimizer(lvl, ProviderType.CPU).optimize(g3)
        assert [n.op_type for n in g3.nodes] == [n.op_type for n in g2.nodes]   # deterministic
    empty = ModelGraph()
    for lvl in ("O0", "O3"):
        Optimizer(lvl).optimize(empty)


def test_gpu_elementwise_chain_fusion_is_semantics_preserving():
    from ronn_b200.graph.passes.provider_specific import GpuOptimizationPass
    b = GraphBuilder().add_input("x", [4, 8]).add_input("z", [4, 8]).add_output("y", [4, 8])
    b.add_op("Relu", ["x"], ["a"]).add_op("Mul", ["a", "z"], ["b"]).add_op("Sigmoid", ["b"], ["c"]).add_op("Add", ["c", "z"], ["y"])
    g = b.build()
    x, z = torch.randn(4, 8), torch.randn(4, 8)
    _, ref = run(g, {"x": x, "z": z})
    g2 = g.clone()
    st = GpuOptimizationPass().run(g2)
    assert st.nodes_fused == 3 and [n.op_type for n in g2.nodes] == ["FusedElementwise"]
    _, out = run(g2, {"x": x, "z": z})
    torch.testing.assert_close(out["y"], ref["y"])


def test_deep_and_wide_graphs():
    b = GraphBuilder().add_input("x", [4]).add_output("t150", [4])
    prev = "x"
    for i in range(1, 151):
        b.add_op("Relu" if i % 2 else "Neg", [prev], [f"t{i}"])
        prev = f"t{i}"
    g = b.build()
    assert g.depth() == 150
    Optimizer("O3", ProviderType.CPU).optimize(g)
    g.validate()
    w = GraphBuilder().add_input("x", [4])
    for i in range(64):
        w.add_op("Relu", ["x"], [f"o{i}"]).add_output(f"o{i}", [4])
    wg = w.build()
    st = Optimizer("O3", ProviderType.CPU).optimize(wg)
    assert len(wg.nodes) == 64 and st.nodes_removed == 0


def test_exact_gelu_is_not_absorbed_into_the_gpu_elementwise_chain():
    import torch
    from ronn_b200.core.types import DataType, ProviderType
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.graph.optimizer import Optimizer
    def build(approx):
        b = GraphBuilder().add_input("x", [2, 8], DataType.F32).add_output("y", [2, 8], DataType.F32)
        b.add_op("Relu", ["x"], ["a"]).add_op("Gelu", ["a"], ["g"], approximate=approx).add_op("Sigmoid", ["g"], ["y"])
        return b.build()
    g_tanh, g_exact = build("tanh"), build("none")
    Optimizer("O3", ProviderType.GPU).optimize(g_tanh)
    Optimizer("O3", ProviderType.GPU).optimize(g_exact)
    assert [n.op_type for n in g_tanh.nodes] == ["FusedElementwise"]
    assert "Gelu" in [n.op_type for n in g_exact.nodes]


def _conv_w(gen, cout, cin):
    return torch.randn(cout, cin, 3, 3, generator=gen) * 0.2


def _check_levels(graph, feeds, names):
    _, ref = run(graph, feeds)
    for lvl in ("O2", "O3"):
        s, out = run(graph, feeds, lvl)
        s.graph().validate()
        node_names = [n.name for n in s.graph().nodes if n.name]
        assert len(node_names) == len(set(node_names))
        for n in names:
            assert out[n].shape == ref[n].shape
            torch.testing.assert_close(out[n], ref[n], atol=1e-4, rtol=1e-4)
    return s


def test_layout_pass_entry_tensor_shared_with_layout_unaware_consumer():
    """A graph input feeds a convolution AND a Concat / Shape: the other consumers keep reading the NCHW tensor."""
    gen = torch.Generator().manual_seed(5)
    b = GraphBuilder().add_input("x", [2, 3, 8, 8]).add_output("y", [2, 6, 8, 8]).add_output("shp", [4])
    b.add_initializer("w1", _conv_w(gen, 3, 3)).add_initializer("w2", _conv_w(gen, 3, 3))
    b.add_op("Conv", ["x", "w1"], ["c1"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("Relu", ["c1"], ["r1"])
    b.add_op("Conv", ["r1", "w2"], ["c2"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("Concat", ["x", "c2"], ["y"], axis=1)
    b.add_op("Shape", ["x"], ["shp"])
    _check_levels(b.build(), {"x": torch.randn(2, 3, 8, 8)}, ["y", "shp"])


def test_layout_pass_non_region_producer_shared_with_outside_consumer():
    """Concat -> three convolutions plus Concat -> Concat: the shared tensor stays NCHW for the outside consumer."""
    gen = torch.Generator().manual_seed(6)
    b = GraphBuilder().add_input("a", [1, 2, 6, 6]).add_input("bb", [1, 2, 6, 6]).add_output("y", [1, 16, 6, 6])
    for i in range(3):
        b.add_initializer(f"w{i}", _conv_w(gen, 4, 4))
    b.add_op("Concat", ["a", "bb"], ["cat"], axis=1)
    for i in range(3):
        b.add_op("Conv", ["cat", f"w{i}"], [f"c{i}"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("Concat", ["cat", "c0", "c1", "c2"], ["y"], axis=1)
    feeds = {"a": torch.randn(1, 2, 6, 6), "bb": torch.randn(1, 2, 6, 6)}
    s = _check_levels(b.build(), feeds, ["y"])
    # the outside Concat still reads the original tensor, not a transposed copy of it
    last = [n for n in s.graph().nodes if n.op_type == "Concat"][-1]
    assert last.inputs[0] == "cat"


def test_layout_pass_tensor_that_is_graph_output_and_read_outside_the_region():
    gen = torch.Generator().manual_seed(7)
    b = GraphBuilder().add_input("x", [2, 3, 8, 8]).add_output("feat", [2, 4, 8, 8]).add_output("flat", [2, 256])
    b.add_initializer("w1", _conv_w(gen, 4, 3)).add_initializer("w2", _conv_w(gen, 4, 4))
    b.add_op("Conv", ["x", "w1"], ["c1"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("Relu", ["c1"], ["r1"])
    b.add_op("Conv", ["r1", "w2"], ["feat"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("Flatten", ["feat"], ["flat"], axis=1)
    s = _check_levels(b.build(), {"x": torch.randn(2, 3, 8, 8)}, ["feat", "flat"])
    back = [n for n in s.graph().nodes if n.op_type == "Transpose" and n.attributes["perm"] == [0, 3, 1, 2]]
    assert len(back) == 1 and back[0].outputs == ["feat"]


def test_qkv_projections_of_an_attention_node_fuse_into_one_gemm():
    from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert
    g = build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=64, n_heads=2, hidden_dim=128), dtype=torch.float32, seed=5)
    ids = torch.randint(0, 512, (3, 10))
    mask = torch.ones(3, 10, dtype=torch.int64)
    mask[1, 6:] = 0
    feeds = {"input_ids": ids, "attention_mask": mask}
    _, ref = run(g, feeds)
    for lvl in ("O2", "O3"):
        s, out = run(g, feeds, lvl)
        torch.testing.assert_close(out["last_hidden_state"], ref["last_hidden_state"], atol=1e-5, rtol=1e-5)
        nodes = s.graph().nodes
        att = [n for n in nodes if n.op_type == "Attention"]
        assert len(att) == 2 and all(n.attr("fused_qkv") == 1 for n in att)
        splits = [n for n in nodes if n.op_type == "Split"]
        assert len(splits) == 2 and all(len(n.outputs) == 3 for n in splits)
        # per layer: one fused QKV projection, the output projection and the two MLP projections
        assert sum(1 for n in nodes if n.op_type == "FusedGemm") == 2 * 4
        w = s.graph().initializers[[n for n in nodes if n.name and n.name.endswith(".qkv")][0].inputs[1]]
        assert tuple(w.shape) == (64, 192)

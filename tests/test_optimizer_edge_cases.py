"""Edge cases of the graph optimiser, at every optimisation level: empty, single-node, disconnected, cyclic, deep, wide,
multi-input / multi-output, diverse and skip-connection graphs; optimising twice changes nothing more; the optimised
graph computes what the original computes (the reference's list: crates/ronn-graph/tests/test_edge_cases.rs:12-460)."""
import pytest
import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.api.errors import RonnError
from ronn_b200.core.types import OptimizationLevel, ProviderType
from ronn_b200.graph.ir import GraphBuilder, ModelGraph
from ronn_b200.graph.optimizer import Optimizer

LEVELS = ["O0", "O1", "O2", "O3"]


def run(graph, feeds, level):
    s = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level(level))
    return s, s.run(feeds)


def check_all_levels(graph, feeds, atol=1e-5):
    _, ref = run(graph, feeds, "O0")
    for lvl in LEVELS[1:]:
        s, out = run(graph, feeds, lvl)
        s.graph().validate()
        assert set(out) == set(ref)
        for k in ref:
            torch.testing.assert_close(out[k], ref[k], atol=atol, rtol=1e-5)
    return ref


@pytest.mark.parametrize("level", LEVELS)
def test_empty_graph(level):
    g = ModelGraph()
    stats = Optimizer(OptimizationLevel.parse(level), ProviderType.CPU).optimize(g)
    assert g.nodes == [] and stats.nodes_removed == 0 and stats.nodes_fused == 0


@pytest.mark.parametrize("level", LEVELS)
def test_single_node_graph(level):
    b = GraphBuilder().add_input("x", [2, 3]).add_output("y", [2, 3])
    b.add_op("Relu", ["x"], ["y"])
    s, out = run(b.build(), {"x": torch.tensor([[-1.0, 0.0, 2.0], [3.0, -4.0, 5.0]])}, level)
    assert [n.op_type for n in s.graph().nodes] == ["Relu"]
    assert out["y"].tolist() == [[0.0, 0.0, 2.0], [3.0, 0.0, 5.0]]


def test_two_disconnected_subgraphs_are_both_kept():
    b = GraphBuilder().add_input("a", [4]).add_input("b", [4]).add_output("ya", [4]).add_output("yb", [4])
    b.add_op("Relu", ["a"], ["ra"]).add_op("Neg", ["ra"], ["ya"])
    b.add_op("Sigmoid", ["b"], ["sb"]).add_op("Tanh", ["sb"], ["yb"])
    check_all_levels(b.build(), {"a": torch.randn(4), "b": torch.randn(4)})


def test_a_disconnected_dead_branch_is_removed_from_o1_on():
    b = GraphBuilder().add_input("a", [4]).add_output("y", [4])
    b.add_op("Relu", ["a"], ["y"]).add_op("Exp", ["a"], ["dead0"]).add_op("Neg", ["dead0"], ["dead1"])
    g = b.build()
    s0, _ = run(g, {"a": torch.randn(4)}, "O0")
    s1, _ = run(g, {"a": torch.randn(4)}, "O1")
    assert len(s0.graph().nodes) == 3 and [n.op_type for n in s1.graph().nodes] == ["Relu"]


@pytest.mark.parametrize("level", LEVELS)
def test_cyclic_graph_is_rejected(level):
    g = ModelGraph()
    from ronn_b200.core.types import DataType
    from ronn_b200.graph.ir import TensorInfo
    g.inputs.append(TensorInfo("x", [2], DataType.F32))
    g.outputs.append(TensorInfo("c", [2], DataType.F32))
    g.add_node("Add", ["x", "c"], ["a"])
    g.add_node("Relu", ["a"], ["b"])
    g.add_node("Neg", ["b"], ["c"])
    with pytest.raises(RonnError, match="[Cc]ycl"):
        g.validate()
    with pytest.raises(RonnError):
        Model.from_graph(g).create_session(SessionOptions().with_optimization_level(level))


def test_graph_without_optimisation_opportunities_is_left_alone():
    b = GraphBuilder().add_input("x", [3, 3]).add_input("z", [3, 3]).add_output("y", [3, 3])
    b.add_op("Transpose", ["x"], ["t"], perm=[1, 0]).add_op("MatMul", ["t", "z"], ["m"]).add_op("Softmax", ["m"], ["y"], axis=-1)
    g = b.build()
    for lvl in LEVELS[:3]:
        s, _ = run(g, {"x": torch.randn(3, 3), "z": torch.randn(3, 3)}, lvl)
        assert [n.op_type for n in s.graph().nodes] == ["Transpose", "MatMul", "Softmax"]
    check_all_levels(g, {"x": torch.randn(3, 3), "z": torch.randn(3, 3)})


@pytest.mark.parametrize("depth", [64, 1500])
def test_very_deep_linear_graph(depth):
    b = GraphBuilder().add_input("x", [8]).add_output(f"t{depth}", [8])
    b.add_initializer("c", torch.full((8,), 0.001))
    prev = "x"
    for i in range(1, depth + 1):
        b.add_op("Add" if i % 2 else "Relu", [prev, "c"] if i % 2 else [prev], [f"t{i}"])
        prev = f"t{i}"
    check_all_levels(b.build(), {"x": torch.randn(8)}, atol=1e-4)


def test_wide_graph_with_many_parallel_branches():
    width = 300
    b = GraphBuilder().add_input("x", [16]).add_output("y", [16])
    for i in range(width):
        b.add_initializer(f"c{i}", torch.full((16,), float(i) / width))
        b.add_op("Mul", ["x", f"c{i}"], [f"m{i}"]).add_op("Relu", [f"m{i}"], [f"r{i}"])
    b.add_op("Sum", [f"r{i}" for i in range(width)], ["y"])
    check_all_levels(b.build(), {"x": torch.randn(16)}, atol=1e-4)


def test_multiple_inputs_and_multiple_outputs():
    b = GraphBuilder().add_input("a", [2, 4]).add_input("b", [2, 4]).add_input("c", [4, 3])
    b.add_output("s", [2, 4]).add_output("p", [2, 3]).add_output("a_again", [2, 4])
    b.add_op("Add", ["a", "b"], ["s"]).add_op("MatMul", ["s", "c"], ["p"]).add_op("Identity", ["a"], ["a_again"])
    ref = check_all_levels(b.build(), {"a": torch.randn(2, 4), "b": torch.randn(2, 4), "c": torch.randn(4, 3)})
    assert set(ref) == {"s", "p", "a_again"}


def test_an_intermediate_that_is_also_a_graph_output_survives_fusion():
    """MatMul -> Add(bias) -> Relu where the pre-activation is a graph output too: the fusion must not swallow it."""
    b = GraphBuilder().add_input("x", [2, 4]).add_output("pre", [2, 3]).add_output("y", [2, 3])
    b.add_initializer("w", torch.randn(4, 3)).add_initializer("bias", torch.randn(3))
    b.add_op("MatMul", ["x", "w"], ["mm"]).add_op("Add", ["mm", "bias"], ["pre"]).add_op("Relu", ["pre"], ["y"])
    check_all_levels(b.build(), {"x": torch.randn(2, 4)})


def test_diverse_operation_types_in_one_graph():
    g = torch.Generator().manual_seed(0)
    b = GraphBuilder().add_input("img", [1, 3, 8, 8]).add_input("vec", [1, 6]).add_output("y", [1, 5])
    b.add_initializer("cw", torch.randn(4, 3, 3, 3, generator=g) * 0.3).add_initializer("gamma", torch.rand(4, generator=g) + 0.5)
    b.add_initializer("beta", torch.randn(4, generator=g)).add_initializer("mean", torch.randn(4, generator=g) * 0.1)
    b.add_initializer("var", torch.rand(4, generator=g) + 0.5).add_initializer("fw", torch.randn(4 + 6, 5, generator=g))
    b.add_initializer("fb", torch.randn(5, generator=g)).add_initializer("two", torch.tensor(2.0))
    b.add_op("Conv", ["img", "cw"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    b.add_op("BatchNormalization", ["c", "gamma", "beta", "mean", "var"], ["bn"]).add_op("Relu", ["bn"], ["r"])
    b.add_op("MaxPool", ["r"], ["mp"], kernel_shape=[2, 2], strides=[2, 2]).add_op("GlobalAveragePool", ["mp"], ["gap"])
    b.add_op("Flatten", ["gap"], ["flat"], axis=1).add_op("Concat", ["flat", "vec"], ["cat"], axis=1)
    b.add_op("Mul", ["cat", "two"], ["sc"]).add_op("Gemm", ["sc", "fw", "fb"], ["lin"]).add_op("Softmax", ["lin"], ["y"], axis=-1)
    check_all_levels(b.build(), {"img": torch.randn(1, 3, 8, 8, generator=g), "vec": torch.randn(1, 6, generator=g)}, atol=1e-4)


@pytest.mark.parametrize("level", LEVELS)
def test_repeated_optimisation_is_stable(level):
    from ronn_b200.models.resnet18 import build_resnet18
    g = build_resnet18(dtype=torch.float32, seed=0, num_classes=10, width=8) if "width" in build_resnet18.__code__.co_varnames \
        else build_resnet18(dtype=torch.float32, seed=0)
    opt = Optimizer(OptimizationLevel.parse(level), ProviderType.CPU)
    opt.optimize(g)
    first = [(n.op_type, tuple(n.inputs), tuple(n.outputs)) for n in g.nodes]
    stats = opt.optimize(g)
    assert [(n.op_type, tuple(n.inputs), tuple(n.outputs)) for n in g.nodes] == first
    assert stats.nodes_fused == 0 and stats.nodes_removed == 0


def test_skip_connection_keeps_both_paths():
    g = torch.Generator().manual_seed(1)
    b = GraphBuilder().add_input("x", [2, 8]).add_output("y", [2, 8])
    b.add_initializer("w1", torch.randn(8, 8, generator=g) * 0.3).add_initializer("b1", torch.randn(8, generator=g))
    b.add_initializer("w2", torch.randn(8, 8, generator=g) * 0.3).add_initializer("b2", torch.randn(8, generator=g))
    b.add_op("MatMul", ["x", "w1"], ["m1"]).add_op("Add", ["m1", "b1"], ["a1"]).add_op("Relu", ["a1"], ["r1"])
    b.add_op("MatMul", ["r1", "w2"], ["m2"]).add_op("Add", ["m2", "b2"], ["a2"]).add_op("Add", ["a2", "x"], ["res"])
    b.add_op("Relu", ["res"], ["y"])
    check_all_levels(b.build(), {"x": torch.randn(2, 8, generator=g)})


def test_executor_releases_intermediates_after_their_last_reader():
    """The kernel compiler's lifetime analysis drives the executor: every intermediate is dropped right after the
    step that reads it last, graph outputs and constants never are, and the results do not change."""
    import gc
    import weakref
    b = GraphBuilder().add_input("x", [4, 8]).add_output("y", [4, 8]).add_output("z", [4, 8])
    b.add_initializer("w", torch.randn(8, 8))
    b.add_op("MatMul", ["x", "w"], ["a"]).add_op("Relu", ["a"], ["r"]).add_op("Add", ["r", "a"], ["s"])
    b.add_op("Tanh", ["s"], ["y"]).add_op("Neg", ["s"], ["z"])
    g = b.build()
    sess = Model.from_graph(g).create_session(SessionOptions().with_optimization_level("O0"))
    k = sess._kernel
    plan = sess.compilation_plan()
    assert plan.groups and plan.memory_plan and plan.peak_bytes > 0
    released = [s for step in k.release_after for s in step]
    assert len(released) == len(set(released)) == 3                      # a, r, s
    assert not set(released) & (set(k.output_slots.values()) | set(k.const_slots) | set(k.input_slots.values()))
    # 'a' is read by Relu and by Add: it must survive until Add (step 2), 'r' too
    names = [st.name for st in k.steps]
    assert [len(step) for step in k.release_after] == [0, 0, 2, 0, 1] or sum(len(s) for s in k.release_after) == 3
    # the dropped tensors really go away: watch them from inside an operator
    seen = []
    real = k.steps[1].fn
    k.steps[1].fn = lambda i, a, c: (seen.append(weakref.ref(i[0])), real(i, a, c))[1]
    x = torch.randn(4, 8)
    out = sess.run({"x": x})
    gc.collect()
    assert seen and seen[0]() is None                                    # 'a' was freed although the outputs are alive
    a = x @ g.initializers["w"]
    s = torch.relu(a) + a
    torch.testing.assert_close(out["y"], torch.tanh(s))
    torch.testing.assert_close(out["z"], -s)

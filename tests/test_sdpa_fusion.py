"""The attention core written in primitives (MatMul -> scale -> mask -> Softmax -> MatMul) becomes one
``com.ronn::ScaledDotProductAttention`` node, and only where that is exact."""
import math

import pytest
import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.graph.ir import GraphBuilder

B, H, S, D = 2, 3, 5, 8


def _core(scale="div", mask=True, scale_after_mask=False, fan_out=False, mask_from_mul=False):
    b = (GraphBuilder().add_input("q", [B, H, S, D]).add_input("kt", [B, H, D, S]).add_input("v", [B, H, S, D])
         .add_output("y", [B, H, S, D]))
    if mask:
        b.add_input("m", [B, 1, 1, S])
    b.add_op("MatMul", ["q", "kt"], ["s0"])
    cur = "s0"

    def add_scale(cur):
        if scale == "div":
            b.add_initializer("c", torch.tensor(math.sqrt(D)))
            b.add_op("Div", [cur, "c"], [cur + "_s"])
        elif scale == "mul":
            b.add_initializer("c", torch.tensor(1.0 / math.sqrt(D)))
            b.add_op("Mul", ["c", cur], [cur + "_s"])
        else:
            return cur
        return cur + "_s"

    def add_mask(cur):
        if not mask:
            return cur
        name = "m"
        if mask_from_mul:
            b.add_initializer("big", torch.tensor(1.0))
            b.add_op("Mul", ["m", "big"], ["m2"])
            name = "m2"
        b.add_op("Add", [cur, name], [cur + "_m"])
        return cur + "_m"

    cur = add_scale(add_mask(cur)) if scale_after_mask else add_mask(add_scale(cur))
    b.add_op("Softmax", [cur], ["p"], axis=-1)
    b.add_op("MatMul", ["p", "v"], ["y"])
    if fan_out:
        b.add_output("p2", [B, H, S, S])
        b.add_op("Identity", ["p"], ["p2"])
    return b.build()


def _feeds(mask=True):
    g = torch.Generator().manual_seed(0)
    f = {"q": torch.randn(B, H, S, D, generator=g), "kt": torch.randn(B, H, D, S, generator=g),
         "v": torch.randn(B, H, S, D, generator=g)}
    if mask:
        m = torch.zeros(B, 1, 1, S)
        m[1, :, :, 3:] = -1e4
        f["m"] = m
    return f


def _ops(graph, level):
    s = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level(level))
    return s, [n.op_type for n in s.graph().nodes]


@pytest.mark.parametrize("scale", ["div", "mul", "none"])
@pytest.mark.parametrize("mask", [True, False])
@pytest.mark.parametrize("mask_from_mul", [False, True])
def test_attention_core_fuses_and_matches(scale, mask, mask_from_mul):
    if mask_from_mul and not mask:
        pytest.skip("no mask")
    g = _core(scale, mask, mask_from_mul=mask_from_mul)
    s0, ops0 = _ops(g, "O0")
    s2, ops2 = _ops(g, "O2")
    assert "Softmax" in ops0 and "ScaledDotProductAttention" not in ops0
    assert ops2.count("ScaledDotProductAttention") == 1 and "Softmax" not in ops2 and "MatMul" not in ops2
    node = next(n for n in s2.graph().nodes if n.op_type == "ScaledDotProductAttention")
    want = {"div": 1.0 / math.sqrt(D), "mul": 1.0 / math.sqrt(D), "none": 1.0}[scale]
    assert abs(float(node.attr("scale")) - want) < 1e-6 and len(node.inputs) == (4 if mask else 3)
    f = _feeds(mask)
    torch.testing.assert_close(s2.run(f)["y"], s0.run(f)["y"], atol=1e-5, rtol=1e-5)
    ref = torch.nn.functional.scaled_dot_product_attention(f["q"], f["kt"].transpose(-1, -2), f["v"],
                                                           attn_mask=f.get("m"), scale=want)
    torch.testing.assert_close(s2.run(f)["y"], ref, atol=1e-5, rtol=1e-5)


def test_a_scale_between_mask_and_softmax_is_left_alone():
    g = _core("div", True, scale_after_mask=True)
    s2, ops2 = _ops(g, "O3")
    assert "ScaledDotProductAttention" not in ops2 and "Softmax" in ops2
    s0, _ = _ops(g, "O0")
    f = _feeds()
    torch.testing.assert_close(s2.run(f)["y"], s0.run(f)["y"], atol=1e-5, rtol=1e-5)


def test_probabilities_with_a_second_reader_are_left_alone():
    g = _core("div", True, fan_out=True)
    s2, ops2 = _ops(g, "O3")
    assert "ScaledDotProductAttention" not in ops2
    s0, _ = _ops(g, "O0")
    f = _feeds()
    out2, out0 = s2.run(f), s0.run(f)
    for k in out0:
        torch.testing.assert_close(out2[k], out0[k], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("scores_first", [False, True])
@pytest.mark.parametrize("additive_too", [False, True])
def test_masked_fill_written_as_where_is_part_of_the_fused_node(scores_first, additive_too):
    b = (GraphBuilder().add_input("q", [B, H, S, D]).add_input("kt", [B, H, D, S]).add_input("v", [B, H, S, D])
         .add_input("keep", [B, 1, 1, S]))
    b.add_output("y", [B, H, S, D])
    b.add_initializer("c", torch.tensor(math.sqrt(D))).add_initializer("neg", torch.tensor(-1e9)).add_initializer("zero", torch.tensor(0.0))
    b.add_op("MatMul", ["q", "kt"], ["s0"]).add_op("Div", ["s0", "c"], ["s1"])
    if scores_first:
        b.add_op("Greater", ["keep", "zero"], ["cond"]).add_op("Where", ["cond", "s1", "neg"], ["s2"])
    else:
        b.add_op("Equal", ["keep", "zero"], ["cond"]).add_op("Where", ["cond", "neg", "s1"], ["s2"])
    cur = "s2"
    if additive_too:
        b.add_input("m", [B, 1, 1, S])
        b.add_op("Add", ["s2", "m"], ["s3"])
        cur = "s3"
    b.add_op("Softmax", [cur], ["p"], axis=-1).add_op("MatMul", ["p", "v"], ["y"])
    g = b.build()
    s0, _ = _ops(g, "O0")
    s2, ops2 = _ops(g, "O2")
    assert ops2.count("ScaledDotProductAttention") == 1 and "Softmax" not in ops2 and "Where" not in ops2
    f = _feeds(additive_too)
    keep = torch.ones(B, 1, 1, S)
    keep[0, :, :, 4:] = 0
    f["keep"] = keep
    torch.testing.assert_close(s2.run(f)["y"], s0.run(f)["y"], atol=1e-5, rtol=1e-5)

"""784-128-10 MLP: MatMul+Add+Relu -> MatMul+Add+Softmax, f32, weights ~N(0, 0.02), zero bias.

The small CPU graph every operator of which the reference implements
(crates/ronn-onnx/src/ops/math.rs:109-131 MatMul, activations.rs:10-114 Relu/Softmax)."""
from __future__ import annotations

import torch

from ..core.types import DataType
from ..graph.ir import GraphBuilder, ModelGraph


def build_mlp784(seed: int = 0, hidden: int = 128, classes: int = 10, in_features: int = 784) -> ModelGraph:
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder()
    b.add_input("input", [1, in_features], DataType.F32)
    b.add_output("probs", [1, classes], DataType.F32)
    b.add_initializer("fc1.weight", torch.randn(in_features, hidden, generator=g) * 0.02)
    b.add_initializer("fc1.bias", torch.zeros(hidden))
    b.add_initializer("fc2.weight", torch.randn(hidden, classes, generator=g) * 0.02)
    b.add_initializer("fc2.bias", torch.zeros(classes))
    b.add_op("MatMul", ["input", "fc1.weight"], ["fc1.mm"], name="fc1_matmul")
    b.add_op("Add", ["fc1.mm", "fc1.bias"], ["fc1.out"], name="fc1_add")
    b.add_op("Relu", ["fc1.out"], ["fc1.act"], name="fc1_relu")
    b.add_op("MatMul", ["fc1.act", "fc2.weight"], ["fc2.mm"], name="fc2_matmul")
    b.add_op("Add", ["fc2.mm", "fc2.bias"], ["fc2.out"], name="fc2_add")
    b.add_op("Softmax", ["fc2.out"], ["probs"], name="softmax", axis=-1)
    graph = b.build()
    graph.metadata["ronn.arch"] = "mlp784"
    return graph

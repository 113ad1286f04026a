"""Small ONNX graphs for examples, fixtures and smoke tests.

Same set as the reference's model scripts: ``scripts/generate_test_model.py:13-124`` (simple add / matmul / relu),
``models/create_test_models.py:11-76,79-148,151-238`` (simple_linear = MatMul + Add, simple_conv = Conv 7x7 / 2 + Relu,
a ResNet-18 *stub* = Conv -> GlobalAveragePool -> Reshape -> MatMul) and
``crates/ronn-api/tests/fixtures/create_fixtures.py:20-104`` (Identity ``simple_model``, ``add_model``).  The graphs are
built with the in-tree graph builder and written with the in-tree ONNX encoder (``Model.save``); no ``onnx`` package.

    python -m ronn_b200.models.test_models out_dir      # writes every model as out_dir/<name>.onnx
"""
from __future__ import annotations

import os
import sys
from typing import Callable, Dict

import torch

from ..core.types import DataType
from ..graph.ir import GraphBuilder, ModelGraph


def simple_model() -> ModelGraph:
    b = GraphBuilder().add_input("input", [1, 3], DataType.F32).add_output("output", [1, 3], DataType.F32)
    return b.add_op("Identity", ["input"], ["output"], name="identity").build()


def simple_add() -> ModelGraph:
    b = GraphBuilder().add_input("a", [1, 4], DataType.F32).add_input("b", [1, 4], DataType.F32)
    b.add_output("sum", [1, 4], DataType.F32)
    return b.add_op("Add", ["a", "b"], ["sum"], name="add").build()


def simple_matmul() -> ModelGraph:
    b = GraphBuilder().add_input("a", [2, 3], DataType.F32).add_input("b", [3, 4], DataType.F32)
    b.add_output("product", [2, 4], DataType.F32)
    return b.add_op("MatMul", ["a", "b"], ["product"], name="matmul").build()


def simple_relu() -> ModelGraph:
    b = GraphBuilder().add_input("x", [1, 8], DataType.F32).add_output("y", [1, 8], DataType.F32)
    return b.add_op("Relu", ["x"], ["y"], name="relu").build()


def simple_linear(in_features: int = 10, out_features: int = 5, seed: int = 0) -> ModelGraph:
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder().add_input("input", [1, in_features], DataType.F32)
    b.add_output("output", [1, out_features], DataType.F32)
    b.add_initializer("weight", torch.randn(in_features, out_features, generator=g) * 0.1)
    b.add_initializer("bias", torch.zeros(out_features))
    b.add_op("MatMul", ["input", "weight"], ["mm"], name="matmul")
    return b.add_op("Add", ["mm", "bias"], ["output"], name="add").build()


def simple_conv(seed: int = 0) -> ModelGraph:
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder().add_input("input", [1, 3, 224, 224], DataType.F32)
    b.add_output("output", [1, 64, 112, 112], DataType.F32)
    b.add_initializer("conv.weight", torch.randn(64, 3, 7, 7, generator=g) * 0.05)
    b.add_op("Conv", ["input", "conv.weight"], ["conv"], name="conv", kernel_shape=[7, 7], strides=[2, 2],
             pads=[3, 3, 3, 3])
    return b.add_op("Relu", ["conv"], ["output"], name="relu").build()


def resnet18_stub(classes: int = 1000, seed: int = 0) -> ModelGraph:
    """Conv -> GlobalAveragePool -> Reshape -> MatMul: the shape of an image classifier without its depth."""
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder().add_input("input", [1, 3, 224, 224], DataType.F32)
    b.add_output("logits", [1, classes], DataType.F32)
    b.add_initializer("conv.weight", torch.randn(64, 3, 7, 7, generator=g) * 0.05)
    b.add_initializer("shape", torch.tensor([1, 64], dtype=torch.int64))
    b.add_initializer("fc.weight", torch.randn(64, classes, generator=g) * 0.05)
    b.add_op("Conv", ["input", "conv.weight"], ["conv"], name="conv", kernel_shape=[7, 7], strides=[2, 2],
             pads=[3, 3, 3, 3])
    b.add_op("GlobalAveragePool", ["conv"], ["pool"], name="pool")
    b.add_op("Reshape", ["pool", "shape"], ["flat"], name="flatten")
    return b.add_op("MatMul", ["flat", "fc.weight"], ["logits"], name="fc").build()


BUILDERS: Dict[str, Callable[[], ModelGraph]] = {
    "simple_model": simple_model, "add_model": simple_add, "simple_add": simple_add, "simple_matmul": simple_matmul,
    "simple_relu": simple_relu, "simple_linear": simple_linear, "simple_conv": simple_conv,
    "resnet18_stub": resnet18_stub,
}


def write_all(out_dir: str) -> Dict[str, str]:
    from ..api.model import Model
    os.makedirs(out_dir, exist_ok=True)
    paths = {}
    for name, build in BUILDERS.items():
        path = os.path.join(out_dir, name + ".onnx")
        Model.from_graph(build()).save(path)
        paths[name] = path
    return paths


if __name__ == "__main__":
    for name, path in write_all(sys.argv[1] if len(sys.argv) > 1 else "models_out").items():
        print(name, path)

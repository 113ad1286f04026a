"""ResNet-18 as a standard-operator ONNX graph with random He-initialised weights
(conv / BatchNormalization / Relu / MaxPool / Add / GlobalAveragePool / Flatten / Gemm-1000; BN mean 0, var 1).

The reference only ships a stub under this name (Conv -> GlobalAveragePool -> Reshape -> MatMul:
models/create_test_models.py:151-238) and cannot execute Conv, BatchNormalization or pooling at all
(crates/ronn-core/src/tensor.rs:330-377)."""
from __future__ import annotations

import math

import torch

from ..core.types import DataType
from ..graph.ir import ModelGraph, TensorInfo


def build_resnet18(num_classes: int = 1000, dtype: torch.dtype = torch.float16, seed: int = 0, batch: int = 0,
                   image: int = 224) -> ModelGraph:
    gen = torch.Generator().manual_seed(seed)
    g = ModelGraph()
    g.name = "resnet18"
    dt = DataType.from_torch(dtype)
    g.inputs.append(TensorInfo("input", [batch, 3, image, image], dt, ["batch" if batch == 0 else None, None, None, None]))
    init = g.initializers

    def conv_bn(x, name, cin, cout, k, stride, pad, relu=True):
        fan_in = cin * k * k
        init[f"{name}.weight"] = (torch.randn(cout, cin, k, k, generator=gen) * math.sqrt(2.0 / fan_in)).to(dtype)
        init[f"{name}.bn.weight"] = torch.ones(cout, dtype=dtype)
        init[f"{name}.bn.bias"] = torch.zeros(cout, dtype=dtype)
        init[f"{name}.bn.running_mean"] = torch.zeros(cout, dtype=dtype)
        init[f"{name}.bn.running_var"] = torch.ones(cout, dtype=dtype)
        g.add_node("Conv", [x, f"{name}.weight"], [f"{name}.conv"],
                   {"kernel_shape": [k, k], "strides": [stride, stride], "pads": [pad] * 4, "dilations": [1, 1], "group": 1},
                   name=f"{name}.conv")
        g.add_node("BatchNormalization", [f"{name}.conv", f"{name}.bn.weight", f"{name}.bn.bias",
                                          f"{name}.bn.running_mean", f"{name}.bn.running_var"], [f"{name}.bn"],
                   {"epsilon": 1e-5}, name=f"{name}.bn")
        if not relu:
            return f"{name}.bn"
        g.add_node("Relu", [f"{name}.bn"], [f"{name}.relu"], name=f"{name}.relu")
        return f"{name}.relu"

    x = conv_bn("input", "stem", 3, 64, 7, 2, 3)
    g.add_node("MaxPool", [x], ["stem.pool"], {"kernel_shape": [3, 3], "strides": [2, 2], "pads": [1, 1, 1, 1]}, name="stem.pool")
    x = "stem.pool"
    cin = 64
    for stage, cout in enumerate((64, 128, 256, 512)):
        for blk in range(2):
            name = f"layer{stage + 1}.{blk}"
            stride = 2 if (stage > 0 and blk == 0) else 1
            y = conv_bn(x, f"{name}.a", cin, cout, 3, stride, 1)
            y = conv_bn(y, f"{name}.b", cout, cout, 3, 1, 1, relu=False)
            skip = x
            if stride != 1 or cin != cout:
                skip = conv_bn(x, f"{name}.down", cin, cout, 1, stride, 0, relu=False)
            g.add_node("Add", [y, skip], [f"{name}.sum"], name=f"{name}.add")
            g.add_node("Relu", [f"{name}.sum"], [f"{name}.out"], name=f"{name}.relu")
            x = f"{name}.out"
            cin = cout
    g.add_node("GlobalAveragePool", [x], ["gap"], name="gap")
    g.add_node("Flatten", ["gap"], ["flat"], {"axis": 1}, name="flatten")
    init["fc.weight"] = (torch.randn(num_classes, 512, generator=gen) * math.sqrt(1.0 / 512)).to(dtype)
    init["fc.bias"] = torch.zeros(num_classes, dtype=dtype)
    g.add_node("Gemm", ["flat", "fc.weight", "fc.bias"], ["logits"], {"transB": 1}, name="fc")
    g.outputs.append(TensorInfo("logits", [batch, num_classes], dt, ["batch" if batch == 0 else None, None]))
    g.metadata.update({"ronn.arch": "resnet18", "ronn.num_classes": str(num_classes)})
    g.validate()
    return g

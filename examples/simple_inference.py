"""Load (or build) an ONNX model, create sessions at two optimisation levels and run them.
Counterpart of the reference's examples/simple-inference and examples/onnx-model."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))      # run from a source checkout

import sys

import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.models.mlp784 import build_mlp784

if len(sys.argv) > 1:
    model = Model.load(sys.argv[1])
else:
    model = Model.from_graph(build_mlp784())
    model.save("/tmp/mlp784.onnx")
    model = Model.load("/tmp/mlp784.onnx")
print(model, model.metadata())
feeds = {i.name: torch.rand([d or 1 for d in i.shape]) for i in model.inputs()}
for level in ("O0", "O3"):
    sess = model.create_session(SessionOptions().with_optimization_level(level).with_provider("cpu"))
    out = sess.run(feeds)
    print(level, {k: tuple(v.shape) for k, v in out.items()}, sess.optimization_stats(), sess.stats())

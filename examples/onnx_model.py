"""Write the small test models as ONNX files, load them back, print their metadata and run them.

Counterpart of the reference's ``examples/onnx-model`` (examples/onnx-model/src/main.rs:14-75), which loads
``simple_{add,matmul,relu}.onnx`` when present and prints inputs, outputs and metadata; here the files are produced
first with the in-tree ONNX encoder, so the example is self-contained."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.models.test_models import write_all

with tempfile.TemporaryDirectory() as d:
    for name, path in write_all(d).items():
        model = Model.load(path)
        ins = [(t.name, t.shape) for t in model.inputs()]
        outs = [(t.name, t.shape) for t in model.outputs()]
        sess = model.create_session(SessionOptions().with_optimization_level("O2").with_provider("cpu"))
        feeds = {n: torch.rand(*[int(s) for s in shape]) for n, shape in ins}
        result = sess.run(feeds)
        print(f"{name:14s} {os.path.getsize(path):8d} bytes  inputs {ins}  outputs {outs}  ->",
              {k: tuple(v.shape) for k, v in result.items()})

"""HRM routing between a BitNet session and a full-precision session, multi-tier memory and continual learning.
Counterpart of the reference's examples/brain-features."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))      # run from a source checkout

import torch

from ronn_b200 import Model
from ronn_b200.hrm import HierarchicalReasoningModule, RoutingStrategy
from ronn_b200.learning import ContinualLearningEngine
from ronn_b200.memory import MultiTierMemory
from ronn_b200.models.mlp784 import build_mlp784

model = Model.from_graph(build_mlp784())
sess = model.create_session(enable_hrm=True)
for name, x in (("small/flat", torch.full((1, 784), 0.5)), ("large/noisy", torch.randn(64, 784) * 4)):
    out = sess.run({"input": x})
    r = sess._router.last
    print(f"{name:12s} -> {r.path_taken.value:8s} score={r.complexity_metrics.complexity_score:.2f} conf={r.confidence:.2f}")

hrm = HierarchicalReasoningModule.with_strategy(RoutingStrategy.ADAPTIVE_HYBRID)
for n in (4, 550, 5000):
    print(n, hrm.process(torch.randn(n)).path_taken.value)

mem = MultiTierMemory()
ids = [mem.store(torch.randn(8), importance=i / 10) for i in range(10)]
print(mem.stats(), mem.consolidate_sync(now=1e12), mem.stats())

eng = ContinualLearningEngine()
x, t = torch.ones(100), torch.full((100,), 2.0)
print([round(eng.learn(x, t).loss, 3) for _ in range(5)])

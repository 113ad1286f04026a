"""Child process: a session built with tp_size = world size (weights sharded by the tensor-parallel graph pass, partial
results summed by AllReduce nodes) against the same session without tensor parallelism."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from ronn_b200 import Model, SessionOptions  # noqa: E402
from ronn_b200.graph.ir import GraphBuilder  # noqa: E402
from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert  # noqa: E402
from ronn_b200.parallel.group import init_distributed  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank, world, _ = init_distributed("gloo", timeout_s=60)
    res = {}
    graph = build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=64, n_heads=4, hidden_dim=128), dtype=torch.float32, seed=5)
    ids = torch.randint(0, 512, (3, 10), generator=torch.Generator().manual_seed(1))
    mask = torch.ones(3, 10, dtype=torch.int64)
    mask[1, 6:] = 0
    feeds = {"input_ids": ids, "attention_mask": mask}
    ref = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level("O0")).run(feeds)["last_hidden_state"]
    for lvl in ("O0", "O3"):
        s = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level(lvl).with_tp_size(world))
        got = s.run(feeds)["last_hidden_state"]
        g = s.graph()
        n_ar = sum(1 for n in g.nodes if n.op_type == "AllReduce")
        full = sum(t.numel() for t in graph.initializers.values() if t.dim() == 2 and t.shape[0] != 512 and t.shape[1] != 512)
        used = {i for n in g.nodes for i in n.inputs}
        mine = sum(t.numel() for k, t in g.initializers.items() if k in used and t.dim() == 2 and 512 not in t.shape)
        res[lvl] = {"err": float((got - ref).abs().max()), "all_reduce_nodes": n_ar, "weight_fraction": mine / full,
                    "tp": g.metadata.get("ronn.tp")}
    # an MLP whose hidden width does not divide by the world size stays replicated (and still correct)
    b = GraphBuilder().add_input("x", [2, 6]).add_output("y", [2, 3])
    gen = torch.Generator().manual_seed(2)
    b.add_initializer("w1", torch.randn(6, 7, generator=gen)).add_initializer("w2", torch.randn(7, 3, generator=gen))
    b.add_op("MatMul", ["x", "w1"], ["h"]).add_op("Relu", ["h"], ["r"]).add_op("MatMul", ["r", "w2"], ["y"])
    g2 = b.build()
    x = torch.randn(2, 6, generator=gen)
    want = Model.from_graph(g2).create_session().run({"x": x})["y"]
    s2 = Model.from_graph(g2).create_session(SessionOptions().with_tp_size(world))
    res["odd"] = {"err": float((s2.run({"x": x})["y"] - want).abs().max()),
                  "all_reduce_nodes": sum(1 for n in s2.graph().nodes if n.op_type == "AllReduce")}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.barrier()


if __name__ == "__main__":
    main()

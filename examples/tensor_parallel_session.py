"""A generic session sharded over the ranks of a process group: SessionOptions.tp_size runs the tensor-parallel graph
pass (column / row parallel MLP pairs and attention heads, AllReduce nodes), every rank keeps 1 / world of the projection
weights and all ranks return the same result.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/tensor_parallel_session.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ronn_b200 import Model, SessionOptions  # noqa: E402
from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert  # noqa: E402
from ronn_b200.parallel.group import init_distributed  # noqa: E402


def main():
    cuda = torch.cuda.is_available()
    rank, world, local = init_distributed("nccl" if cuda else "gloo", timeout_s=120)
    graph = build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=128, n_heads=4, hidden_dim=256), dtype=torch.float32, seed=5)
    ids = torch.randint(0, 512, (2, 16), generator=torch.Generator().manual_seed(1))
    feeds = {"input_ids": ids, "attention_mask": torch.ones(2, 16, dtype=torch.int64)}
    whole = Model.from_graph(graph).create_session(SessionOptions()).run(feeds)["last_hidden_state"]
    sess = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level("O3").with_tp_size(world))
    part = sess.run(feeds)["last_hidden_state"]
    g = sess.graph()
    n_ar = sum(1 for n in g.nodes if n.op_type == "AllReduce")
    if rank == 0:
        print(f"world {world}: {n_ar} AllReduce nodes, max |diff| vs the unsharded session = {float((part - whole).abs().max()):.2e}")
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

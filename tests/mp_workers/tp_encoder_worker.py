"""Child process: tensor-parallel EncoderRunner (library collectives on CPU ranks) against the single-rank runner."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert  # noqa: E402
from ronn_b200.parallel.group import TPComm, init_distributed  # noqa: E402
from ronn_b200.serving.encoder_runner import EncoderRunner  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank, world, local = init_distributed("gloo", timeout_s=120)
    graph = build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=128, n_heads=4, hidden_dim=256), dtype=torch.float32, seed=11)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 512, (3, 24), generator=g)
    mask = torch.ones(3, 24, dtype=torch.int64)
    mask[1, 15:] = 0
    tp = EncoderRunner(graph, device="cpu", comm=TPComm()).forward(ids, mask)
    single = EncoderRunner(graph, device="cpu").forward(ids, mask)
    sp = EncoderRunner(graph, device="cpu", comm=TPComm(), sequence_parallel=True).forward(ids, mask)
    err, err_sp = 0.0, 0.0
    for b, n in enumerate(mask.sum(1).tolist()):
        err = max(err, (tp[b, :n] - single[b, :n]).abs().max().item())
        err_sp = max(err_sp, (sp[b, :n] - single[b, :n]).abs().max().item())
    gathered = [None] * world
    torch.distributed.all_gather_object(gathered, tp[0, :5, :8].tolist())
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"world": world, "err": err, "err_sequence_parallel": err_sp, "same_across_ranks": all(x == gathered[0] for x in gathered)}, f)
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

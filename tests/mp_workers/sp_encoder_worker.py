"""Child process (one per GPU): the sequence-parallel EncoderRunner on the fused kernels (all-gather inside the
column-parallel GEMM, reduce-scatter inside the row-parallel GEMM) against the single-GPU runner."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert  # noqa: E402
from ronn_b200.parallel import make_comm  # noqa: E402
from ronn_b200.parallel.group import init_distributed  # noqa: E402
from ronn_b200.serving.encoder_runner import EncoderRunner  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank, world, local = init_distributed("nccl", timeout_s=120)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    graph = build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=512, n_heads=8, hidden_dim=1024,
                                                   max_position_embeddings=128), dtype=torch.bfloat16,
                             seed=11)
    g = torch.Generator().manual_seed(2)
    B, S = 8, 128
    ids = torch.randint(0, 512, (B, S), generator=g).to(dev)
    mask = torch.ones(B, S, dtype=torch.int64, device=dev)
    mask[1, 90:] = 0
    mask[6, 5:] = 0
    comm = make_comm("fused", dev)
    sp = EncoderRunner(graph, device=dev, comm=comm, sequence_parallel=True)
    calls0 = comm.fused_calls
    got = sp.forward(ids, mask)
    comm.check()
    fused_calls = comm.fused_calls - calls0
    want = EncoderRunner(graph, device=dev).forward(ids, mask)
    err = 0.0
    for b, n in enumerate(mask.sum(1).tolist()):
        err = max(err, (got[b, :n].float() - want[b, :n].float()).abs().max().item())
    gathered = [None] * world
    torch.distributed.all_gather_object(gathered, got[0, :5, :8].float().tolist())
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"world": world, "err": err, "fused_calls": fused_calls,
                       "same_across_ranks": all(x == gathered[0] for x in gathered)}, f)
    torch.distributed.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)            # symmetric-memory teardown after fused kernels can stall interpreter exit


if __name__ == "__main__":
    main()

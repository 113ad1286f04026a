"""Kernel timeline of one tensor-parallel decode step on rank 0, from the PyTorch profiler (CUPTI activity records).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ronn_b200.parallel.step_timeline

`ncu` cannot wrap a multi-rank run, and per-kernel CUDA events would break the step's CUDA graph; the profiler's
activity records give the start and the duration of every kernel of a replayed graph without either.  With
programmatic dependent launch a kernel is resident while it still waits for its predecessor, so durations overlap:
``RONN_PDL=0`` gives durations that add up to the step.  The numbers are for analysis (which kernels make up a step),
not benchmark values: those come from ``bench.py``.

The reference has no counterpart (its tracing is host-side spans, crates/ronn-core/src/logging.rs).
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import sys


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--decode-steps", type=int, default=140, help="decode steps before the profiled ones")
    ap.add_argument("--show", type=int, default=16, help="kernels of the step's timeline to print")
    args = ap.parse_args()
    import torch
    from torch.profiler import ProfilerActivity, profile
    from ..api.model import Model
    from ..models.gpt2 import GPT2Config, build_gpt2
    from ..serving import EngineConfig, LLMEngine, SamplingParams
    from .group import init_distributed

    rank, world, local = init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    model = Model.from_graph(build_gpt2(GPT2Config(n_layer=args.layers), dtype=torch.bfloat16, seed=0, with_lm_head=False))
    ecfg = EngineConfig(max_num_seqs=args.requests, max_batch_tokens=8192, max_model_len=1024, dtype="bf16",
                        backend="kernels", use_cuda_graph=True, tp_size=world, tp_comm="fused",
                        num_blocks=args.requests * 50)
    comm = None
    if world > 1:
        from . import make_comm
        comm = make_comm("fused", dev)
    eng = LLMEngine(model, ecfg, device=dev, comm=comm)
    g = torch.Generator().manual_seed(0)
    for _ in range(args.requests):
        n = int(torch.randint(64, 513, (1,), generator=g))
        eng.add_request(torch.randint(0, 50257, (n,), generator=g).tolist(),
                        SamplingParams(max_new_tokens=args.decode_steps + 60))
    for _ in range(args.decode_steps):
        eng.step()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    steps = 4
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            eng.step()
        torch.cuda.synchronize()
    if rank == 0:
        evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        evs.sort(key=lambda e: e.time_range.start)
        n = len(evs) // steps
        last = evs[-n:]                                   # the last profiled step
        span = last[-1].time_range.end - last[0].time_range.start
        busy = sum(e.time_range.end - e.time_range.start for e in last)
        per = collections.OrderedDict()
        for e in last:
            d = per.setdefault(e.name[:72], [0, 0.0])
            d[0] += 1
            d[1] += e.time_range.end - e.time_range.start
        print(json.dumps({"world": world, "pdl": os.environ.get("RONN_PDL", "1") != "0", "records_in_step": n,
                          "span_us": round(span, 1), "sum_of_durations_us": round(busy, 1)}))
        print("per kernel (total us, launches, us per launch):")
        for k, (c, t) in sorted(per.items(), key=lambda kv: -kv[1][1])[:10]:
            print(f"{t:9.1f}  x{c:4d}  {t / c:7.2f}  {k}")
        first = min(8, max(n - args.show - 1, 0))
        base = last[first].time_range.start
        print(f"timeline of records {first}..{first + args.show} (start offset us, duration us, start of the next one after us):")
        for i in range(first, min(first + args.show, n - 1)):
            e = last[i]
            print(f"  +{e.time_range.start - base:7.1f}  {e.time_range.end - e.time_range.start:6.1f}  "
                  f"{last[i + 1].time_range.start - e.time_range.start:6.1f}  {e.name[:56]}")
    sys.stdout.flush()
    torch.cuda.synchronize()
    if world > 1:
        os._exit(0)            # symmetric-memory teardown after fused kernels can stall interpreter exit
    return 0


if __name__ == "__main__":
    sys.exit(main())

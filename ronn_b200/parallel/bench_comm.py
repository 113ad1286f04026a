"""Micro-benchmark of the fused row-parallel GEMM + collective against the library composition.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m ronn_b200.parallel.bench_comm

For the decode shapes of GPT-2 medium at this world size it times, per call (CUDA-graph replay of 20 back-to-back
calls, device events, max over ranks):
  fused      ONE kernel: partial GEMM + cross-rank reduction over NVLink + bias + residual + LayerNorm
  library    tcgen05 GEMM kernel + NCCL all-reduce + torch add(bias, residual) + LayerNorm kernel
  gemm_only  the local partial GEMM alone (lower bound of both)
and reports the roofline of the fused op: max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s).
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .group import TPComm, init_distributed
from .symm import FusedComm


def _time_graph(fn, reps=20, iters=5):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps)
    ts.sort()
    return ts[len(ts) // 2]


def main():
    rank, world, local = init_distributed("nccl", timeout_s=120)
    dev = torch.device("cuda", local)
    comm = FusedComm(dev, max_rows=8192, max_cols=1024)
    lib = TPComm()
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")) as f:
            tf = json.load(f)["bf16_tflops"]
    except Exception:
        tf = 1590.0
    out = []
    for (M, N, Kfull, name) in [(256, 1024, 1024, "attn-out"), (256, 1024, 4096, "mlp-down"), (8192, 1024, 1024, "attn-out prefill"),
                                (8192, 1024, 4096, "mlp-down prefill")]:
        Kl = Kfull // world
        a = torch.randn(M, Kl, device=dev).bfloat16()
        w = (torch.randn(N, Kl, device=dev) * 0.05).bfloat16()
        bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
        res = torch.randn(M, N, device=dev).bfloat16()
        gam = torch.ones(N, device=dev, dtype=torch.bfloat16)

        def fused():
            comm.gemm_allreduce(a, w, bias, res, norm=("layernorm", gam, bias, 1e-5))

        def library():
            y = K.gemm(a, w)
            lib.all_reduce(y)
            y = y + bias + res
            K.layernorm(y, gam, bias, 1e-5)

        def gemm_only():
            K.gemm(a, w)

        t_f, t_l, t_g = _time_graph(fused), _time_graph(library), _time_graph(gemm_only)
        t_f, t_l, t_g = lib.max_over_ranks(t_f), lib.max_over_ranks(t_l), lib.max_over_ranks(t_g)
        flops = 2.0 * M * N * Kl
        nvlink_bytes = (world - 1) * M * N * 2.0                 # each rank pulls every peer's bf16 partials
        roof = max(flops / (tf * 1e12), nvlink_bytes / 770e9) * 1e6
        out.append({"op": name, "M": M, "N": N, "K_local": Kl, "world": world, "fused_us": round(t_f, 2),
                    "library_us": round(t_l, 2), "gemm_only_us": round(t_g, 2), "roofline_us": round(roof, 2),
                    "fused_frac_of_roofline": round(roof / t_f, 3), "speedup_vs_library": round(t_l / t_f, 2)})
    comm.check()
    if rank == 0:
        for r in out:
            print(json.dumps(r))
    sys.stdout.flush()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()

"""Micro-benchmark of the fused row-parallel GEMM + collective against the library composition.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m ronn_b200.parallel.bench_comm

For the decode shapes of GPT-2 medium at this world size it times, per call (CUDA-graph replay of 20 back-to-back
calls, device events, max over ranks):
  fused      ONE kernel: partial GEMM + cross-rank reduction over NVLink + bias + residual + LayerNorm, once per
             exchange protocol (two-shot over NVLS multimem, two-shot over peer loads / stores, one-shot pull)
  library    tcgen05 GEMM kernel + NCCL all-reduce + torch add(bias, residual) + LayerNorm kernel
  gemm_only  the local partial GEMM alone (lower bound of both)
and reports the roofline of the fused op: max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s), with the
bytes of a minimal all-reduce, 2 (W - 1) / W x result, which is what the two-shot protocol moves.

For the low-latency and two-shot protocols it also prints where the time of one call goes: %globaltimer stamps taken inside the kernel
(entry, GEMM stored, counters raised, all ranks' tiles seen, rows reduced and stored, "delivered" raised, all
deliveries seen), median over the CTAs of a rank, then the max over ranks.

``--sequence-parallel`` times only the two kernels of the token-sharded layout (gather inside the column-parallel GEMM,
reduce-scatter inside the row-parallel GEMM) at prefill size; ``--all`` adds them to the list above.
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


def sequence_parallel_rows(comm, lib, dev, world, tf):
    """The two fused kernels of the token-sharded layout at GPT-2-medium prefill size (8192 tokens): the gather inside
    the column-parallel GEMM (``ag_gemm``) and the reduce-scatter inside the row-parallel GEMM, against all-gather /
    reduce-scatter calls around the same tcgen05 GEMM.  The shard buffer is single-buffered, so a gather is timed
    together with the reduce-scatter that has to follow it; the gather's own time is the difference."""
    T, H = 8192, 1024
    per = T // world
    x_local = torch.randn(per, H, device=dev).bfloat16()
    w_col = (torch.randn(3 * H // world, H, device=dev) * 0.05).bfloat16()            # QKV, column shard
    att = torch.randn(T, H // world, device=dev).bfloat16()
    w_row = (torch.randn(H, H // world, device=dev) * 0.05).bfloat16()                # out-projection, row shard
    bias = torch.zeros(H, device=dev, dtype=torch.bfloat16)
    res = torch.randn(per, H, device=dev).bfloat16()
    shard = comm.shard_buffer(per, H)

    def fused_rs():
        comm.gemm_reduce_scatter(att, w_row, bias, res)

    def fused_pair():
        shard.copy_(x_local)
        comm.signal_shard_ready()
        comm.ag_gemm(per, H, w_col)
        comm.gemm_reduce_scatter(att, w_row, bias, res)

    def lib_rs():
        lib.reduce_scatter_rows(K.gemm(att, w_row)) + bias + res

    def lib_pair():
        K.gemm(lib.all_gather_rows(x_local), w_col)
        lib.reduce_scatter_rows(K.gemm(att, w_row)) + bias + res

    t = {k: lib.max_over_ranks(_time_graph(f, reps=10)) for k, f in
         (("fused_rs", fused_rs), ("fused_pair", fused_pair), ("lib_rs", lib_rs), ("lib_pair", lib_pair))}
    link = (world - 1) / world * T * H * 2.0 / 770e9 * 1e6                              # one shard set over NVLink, 16-bit
    roof_ag = max(2.0 * T * (3 * H // world) * H / (tf * 1e12) * 1e6, link)
    roof_rs = max(2.0 * T * H * (H // world) / (tf * 1e12) * 1e6, link)
    ag_f, ag_l = t["fused_pair"] - t["fused_rs"], t["lib_pair"] - t["lib_rs"]
    return [{"op": "ag_gemm (QKV, token-sharded input)", "tokens": T, "N_local": 3 * H // world, "K": H, "world": world,
             "fused_us": round(ag_f, 2), "library_us": round(ag_l, 2), "roofline_us": round(roof_ag, 2),
             "fused_frac_of_roofline": round(roof_ag / max(ag_f, 1e-3), 3)},
            {"op": "gemm + reduce-scatter (attention output)", "tokens": T, "N": H, "K_local": H // world, "world": world,
             "fused_us": round(t["fused_rs"], 2), "library_us": round(t["lib_rs"], 2), "roofline_us": round(roof_rs, 2),
             "fused_frac_of_roofline": round(roof_rs / t["fused_rs"], 3)}]


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
    only_sp = "--sequence-parallel" in sys.argv
    if only_sp or "--all" in sys.argv:
        out += sequence_parallel_rows(comm, lib, dev, world, tf)
    for (M, N, Kfull, name) in [] if only_sp else [(256, 1024, 1024, "attn-out"), (256, 1024, 4096, "mlp-down"), (8192, 1024, 1024, "attn-out prefill"),
                                (8192, 1024, 4096, "mlp-down prefill")]:
        Kl = Kfull // world
        a = torch.randn(M, Kl, device=dev).bfloat16()
        w = (torch.randn(N, Kl, device=dev) * 0.05).bfloat16()
        bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
        res = torch.randn(M, N, device=dev).bfloat16()
        gam = torch.ones(N, device=dev, dtype=torch.bfloat16)

        def fused():
            comm.gemm_allreduce(a, w, bias, res, norm=("layernorm", gam, bias, 1e-5))

        def phases():
            """One eager call with in-kernel timestamps: ns spent per phase (median over CTAs)."""
            tr = torch.zeros((600, 8), dtype=torch.int64, device=dev)
            comm.trace = tr
            dist.barrier()
            torch.cuda.synchronize()
            fused()
            torch.cuda.synchronize()
            comm.trace = None
            t = tr[tr[:, 0] > 0].double()
            if t.numel() == 0:
                return {}
            t0 = t[:, 0].min()
            med = lambda col: float((t[:, col][t[:, col] > 0] - t0).median().item()) if bool((t[:, col] > 0).any()) else 0.0
            if comm.proto == "ll":
                marks = {"partials_sent": med(1), "owned_rows_broadcast": med(3), "all_rows_normalised": med(4),
                         "exit": float((t[:, 7].max() - t0).item())}
            else:
                marks = {"gemm_stored": med(1), "published": med(2), "all_tiles_seen": med(3), "rows_stored": med(4),
                         "delivered_sent": med(5), "all_delivered_seen": med(6), "exit": float((t[:, 7].max() - t0).item())}
            return {k: round(lib.max_over_ranks(v) / 1e3, 2) for k, v in marks.items()}

        def library():
            y = K.gemm(a, w)
            lib.all_reduce(y)
            y = y + bias + res
            K.layernorm(y, gam, bias, 1e-5)

        def gemm_only():
            K.gemm(a, w)

        t_l, t_g = lib.max_over_ranks(_time_graph(library)), lib.max_over_ranks(_time_graph(gemm_only))
        flops = 2.0 * M * N * Kl
        # per GPU and direction: fp32 partials of the rows it owns come in from W - 1 peers (1/W of the result each),
        # the finished 16-bit rows (X and H) go out to W - 1 peers
        nvlink_bytes = (world - 1) / world * M * N * (4.0 + 2 * 2.0)
        roof = max(flops / (tf * 1e12), nvlink_bytes / 770e9) * 1e6
        row = {"op": name, "M": M, "N": N, "K_local": Kl, "world": world, "library_us": round(t_l, 2),
               "gemm_only_us": round(t_g, 2), "roofline_us": round(roof, 2)}
        have_mc = comm.nvls_available and os.environ.get("RONN_NVLS", "1") != "0"
        protos = []
        if comm._ll_ok(M, N):
            protos += ([("ll_nvls", "ll", True)] if have_mc else []) + [("ll_p2p", "ll", False)]
        protos += ([("two_shot_nvls", "two_shot", True)] if have_mc else []) + [("two_shot_p2p", "two_shot", False)]
        if M * N <= comm.one_shot_elems:
            protos.append(("one_shot_pull", "pull", False))
        for tag, proto, nvls in protos:
            comm.proto, comm.nvls, comm.push = proto, nvls, False
            t_f = lib.max_over_ranks(_time_graph(fused))
            row[tag + "_us"] = round(t_f, 2)
            row[tag + "_frac_of_roofline"] = round(roof / t_f, 3)
            row[tag + "_speedup_vs_library"] = round(t_l / t_f, 2)
            if proto in ("two_shot", "ll"):
                row[tag + "_phases_us"] = phases()
        out.append(row)
    comm.check()
    if rank == 0:
        for r in out:
            print(json.dumps(r))
    sys.stdout.flush()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()

"""Kernel micro-benchmarks with CUDA-event timing and roofline accounting.

    python -m ronn_b200.ops.microbench gemm --m 256 --n 1024 --k 1024
    python -m ronn_b200.ops.microbench attention --batch 256 --ctx 416 --heads 16 --dim 64
    python -m ronn_b200.ops.microbench decode-shapes          # every GEMM / attention shape of a GPT-2-medium decode step

Timing: warm-up, then ``iters`` launches between two events on the launching stream with an L2 flush
(a 256 MB write) before each timed launch unless ``--no-flush``; reports the median.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

from . import kernels as K


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


_FLUSH = None


def time_kernel(fn, iters=20, warmup=5, flush=True):
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _FLUSH.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def time_graph(make_call, variants: int, reps: int = 40, iters: int = 5):
    """Median time per launch of `reps` back-to-back launches replayed from a CUDA graph.  `make_call(i)` launches
    the kernel on the i-th of `variants` operand sets (rotating operand sets larger than L2 keep DRAM traffic real)."""
    for i in range(min(variants, 3)):
        make_call(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for r in range(reps):
            make_call(r % variants)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps)
    ts.sort()
    return ts[len(ts) // 2]


def bench_dense_attention(batch=64, seq=128, heads=12, dim=64, causal=False, iters=20, flush=True):
    """Tensor-core attention over a fused qkv buffer of `batch` sequences of `seq` tokens.  Timed as back-to-back
    launches replayed from a CUDA graph over rotating operand sets that together exceed L2 (a single eager launch of
    a 20-50 us kernel measures the host's launch path as much as the kernel); ``flush=False`` keeps one operand set."""
    hn = heads * dim
    per_set = batch * seq * hn * 8
    nvar = max(2, int(400e6 // per_set) + 1) if flush else 1
    qkvs = [torch.randn(batch * seq, 3 * hn, device="cuda").bfloat16() for _ in range(nvar)]
    outs = [torch.empty(batch * seq, hn, device="cuda", dtype=torch.bfloat16) for _ in range(nvar)]
    plan = K.dense_attention_plan([seq] * batch, "cuda")
    us = time_graph(lambda i: K.dense_attention(qkvs[i], 0, hn, 2 * hn, plan, heads, heads, dim, causal, out=outs[i]),
                    nvar, reps=max(nvar, 20), iters=max(3, iters // 4))
    K.check_status()
    hbm, tf, src = _peaks()
    flops = 4.0 * batch * heads * seq * seq * dim * (0.5 if causal else 1.0)
    byts = 2.0 * (qkvs[0].numel() + outs[0].numel())
    roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e6
    return {"kernel": "dense_attention", "batch": batch, "seq": seq, "heads": heads, "dim": dim,
            "causal": causal, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "roofline_us": round(roof, 2),
            "frac_of_" + src: round(roof / us, 3), "timing": "CUDA-graph replay, %d operand sets" % nvar}


def bench_fused_single_rank(m=256, n=1024, k=1024, iters=20, flush=True):
    """The fused GEMM + reduction (+ LayerNorm) kernel run as a world of one rank on plain device buffers: the same
    code path as the tensor-parallel call (partials published, flags raised and awaited, rows reduced and normalised)
    without a peer, for profiling on a single GPU."""
    import ctypes as C
    from .. import _native
    a = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias, gamma, beta = (torch.randn(n, device="cuda").bfloat16() for _ in range(3))
    res = torch.randn(m, n, device="cuda").bfloat16()
    stride = m * n * 2
    part = torch.zeros(2 * stride, dtype=torch.uint8, device="cuda")
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    state = torch.zeros(8, dtype=torch.int32, device="cuda")
    out, normed = torch.empty_like(res), torch.empty_like(res)
    pp = (C.c_void_p * 8)(*[part.data_ptr()] + [None] * 7)
    fp = (C.c_void_p * 8)(*[flags.data_ptr()] + [None] * 7)
    lib = _native.cuda()

    def call():
        rc = lib.ronn_gemm_reduce(a.data_ptr(), w.data_ptr(), m, n, k, k, k, pp, fp, stride, state.data_ptr(), 0, 1, 0, m,
                                  out.data_ptr(), n, bias.data_ptr(), res.data_ptr(), n, 2.0, 0, 0, normed.data_ptr(),
                                  gamma.data_ptr(), beta.data_ptr(), 1e-5, 1, K.status_word("cuda").data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
    us = time_kernel(call, iters=iters, flush=flush)
    K.check_status()
    ref = a.float() @ w.float().t()
    ref = ref.bfloat16().float() + bias.float() + res.float()
    err = (out.float() - ref).abs().max().item()
    us_plain = time_kernel(lambda: K.layernorm(K.gemm(a, w, bias, res), gamma, beta, 1e-5), iters=iters, flush=flush)
    return {"kernel": "gemm_reduce(world=1)+layernorm", "m": m, "n": n, "k": k, "us": round(us, 2),
            "gemm_then_layernorm_us": round(us_plain, 2), "max_abs_err": round(err, 4)}


def bench_gemm(m, n, k, dtype=torch.bfloat16, bn=0, act="", flush=True, iters=20):
    a = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(dtype)
    out = torch.empty(m, n, device="cuda", dtype=dtype)
    us = time_kernel(lambda: K.gemm(a, w, activation=act, out=out, bn=bn), iters=iters, flush=flush)
    K.check_status()
    hbm, tf, src = _peaks()
    flops = 2.0 * m * n * k
    byts = 2.0 * (m * k + n * k + m * n)
    t_roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e6
    res = {"kernel": "gemm", "m": m, "n": n, "k": k, "bn": bn, "us": round(us, 2),
           "tflops": round(flops / us / 1e6, 1), "gbs": round(byts / us / 1e3, 1),
           "roofline_us": round(t_roof, 2), "frac_of_" + src: round(t_roof / us, 3)}
    if m <= 1024:
        # a single launch of a few microseconds is dominated by the host's launch latency (the GPU idles between the
        # start event and the kernel): also report back-to-back launches replayed from a CUDA graph, weights rotating
        # through more than L2
        nvar = max(2, int(300e6 // (n * k * 2)))
        ws = [w] + [(torch.randn(n, k, device="cuda") * 0.05).to(dtype) for _ in range(nvar - 1)]
        res["graph_us"] = round(time_graph(lambda i: K.gemm(a, ws[i], activation=act, out=out, bn=bn), nvar), 2)
    return res


def bench_attention(batch, ctx, heads, dim, kv_heads=None, dtype=torch.bfloat16, flush=True, iters=20, ragged=False,
                    splits=None):
    """Decode attention over a paged cache.  ``ragged``: context lengths uniform in [ctx / 4, 7 ctx / 4] (mean ctx)
    instead of all equal.  Timed as a CUDA-graph replay over caches that together exceed L2."""
    kv_heads = kv_heads or heads
    gen = torch.Generator().manual_seed(0)
    lens_h = torch.randint(max(ctx // 4, 1), 7 * ctx // 4 + 1, (batch,), generator=gen) if ragged else torch.full((batch,), ctx)
    max_len = int(lens_h.max())
    nb_seq = (max_len + 15) // 16
    nblocks = batch * nb_seq
    per_set = 2 * nblocks * kv_heads * 16 * dim * 2
    nvar = max(2, int(400e6 // per_set) + 1) if flush else 1
    kcs = [torch.randn(nblocks, kv_heads, 16, dim, device="cuda").to(dtype) for _ in range(nvar)]
    vcs = [torch.randn(nblocks, kv_heads, 16, dim, device="cuda").to(dtype) for _ in range(nvar)]
    bt = torch.randperm(nblocks, device="cuda").to(torch.int32).reshape(batch, nb_seq)
    q = torch.randn(batch, heads * dim, device="cuda").to(dtype)
    lens = lens_h.to("cuda", torch.int32)
    out = torch.empty(batch, heads * dim, device="cuda", dtype=dtype)
    mc = -(-max_len // 16) * 16
    sp = splits if splits else K.attention_splits(batch, heads, mc)
    us = time_graph(lambda i: K.paged_attention(q, kcs[i], vcs[i], bt, lens, heads, kv_heads, dim, max_ctx=mc, out=out,
                                                splits=sp), nvar, reps=max(nvar, 20), iters=max(3, iters // 4))
    hbm, tf, src = _peaks()
    byts = 2.0 * float(lens_h.sum()) * kv_heads * dim * 2
    t_roof = byts / (hbm * 1e9) * 1e6
    return {"kernel": "paged_attention", "batch": batch, "ctx": ctx, "ragged": bool(ragged), "heads": heads, "dim": dim,
            "splits": sp, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1), "roofline_us": round(t_roof, 2),
            "frac_of_" + src: round(t_roof / us, 3)}


def bench_norm(rows, h, dtype=torch.bfloat16, flush=True):
    x = torch.randn(rows, h, device="cuda").to(dtype)
    g = torch.ones(h, device="cuda", dtype=dtype)
    b = torch.zeros(h, device="cuda", dtype=dtype)
    us = time_kernel(lambda: K.layernorm(x, g, b), flush=flush)
    hbm, _, src = _peaks()
    byts = 2.0 * rows * h * 2
    return {"kernel": "layernorm", "rows": rows, "h": h, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1),
            "frac_of_" + src: round(byts / (hbm * 1e9) * 1e6 / us, 3)}


def bench_memory_kernels(flush=True):
    """Every memory-bound kernel of the library on operands larger than L2: time, algorithmic bytes and the fraction
    of the copy bandwidth.  Shapes are the serving shapes widened in the row count until DRAM traffic is real."""
    from . import bitnet as B
    from ..providers.gpu_conv import maxpool_nhwc, global_avgpool_nhwc
    hbm, _, src = _peaks()
    dev, bf = "cuda", torch.bfloat16
    out = []

    def row(name, shape, byts, fn):
        us = time_kernel(fn, flush=flush)
        out.append({"kernel": name, "shape": shape, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1),
                    "frac_of_" + src: round(byts / (hbm * 1e9) * 1e6 / us, 3)})

    R, H = 131072, 1024
    x = torch.randn(R, H, device=dev).to(bf)
    r = torch.randn(R, H, device=dev).to(bf)
    g, b = torch.ones(H, device=dev, dtype=bf), torch.zeros(H, device=dev, dtype=bf)
    row("layernorm", [R, H], 2.0 * R * H * 2, lambda: K.layernorm(x, g, b))
    row("layernorm + residual (sum kept)", [R, H], 4.0 * R * H * 2, lambda: K.layernorm(x, g, b, residual=r, return_sum=True))
    row("rmsnorm", [R, H], 2.0 * R * H * 2, lambda: K.rmsnorm(x, g))
    row("softmax", [R, H], 2.0 * R * H * 2, lambda: K.softmax(x))
    row("gelu", [R, H], 2.0 * R * H * 2, lambda: K.unary(x, "gelu"))
    row("relu", [R, H], 2.0 * R * H * 2, lambda: K.unary(x, "relu"))
    row("sigmoid", [R, H], 2.0 * R * H * 2, lambda: K.unary(x, "sigmoid"))
    row("add", [R, H], 3.0 * R * H * 2, lambda: K.binary(x, r, "add"))
    row("swiglu (gate | up in one buffer)", [R, H], 1.5 * R * H * 2, lambda: K.swiglu_fused(x))
    row("cast bf16 -> fp32", [R, H], 3.0 * R * H * 2, lambda: K.cast(x, torch.float32))
    Hq = 2560
    xq = torch.randn(65536, Hq, device=dev).to(bf)
    gq = torch.ones(Hq, device=dev, dtype=bf)
    row("act_quant_int8", [65536, Hq], 65536.0 * Hq * 3, lambda: B.act_quant_int8(xq))
    row("rmsnorm + act_quant_int8", [65536, Hq], 65536.0 * Hq * 3, lambda: B.rmsnorm_quant_int8(xq, gq))
    V = 50264
    table = torch.randn(V, H, device=dev).to(bf)
    ptab = torch.randn(1024, H, device=dev).to(bf)
    ids = torch.randint(0, V, (R,), device=dev, dtype=torch.int32)
    pos = torch.randint(0, 1024, (R,), device=dev, dtype=torch.int32)
    row("embedding gather + position add", [R, H], 3.0 * R * H * 2, lambda: K.embedding(ids, table, pos, ptab))
    logits = torch.randn(2048, V, device=dev).to(bf)
    row("argmax over the vocabulary", [2048, V], 2048.0 * V * 2, lambda: K.argmax(logits))
    heads, d, T = 16, 64, 65536
    qkv = torch.randn(T, 3 * heads * d, device=dev).to(bf)
    kc = torch.zeros(T // 16 + 1, heads, 16, d, device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(T, device=dev).to(torch.int32)
    row("kv_append (paged scatter)", [T, heads, d], 4.0 * T * heads * d * 2,
        lambda: K.kv_append(qkv, heads * d, 2 * heads * d, slots, kc, vc, heads, heads, d))
    xi = torch.randn(128, 112, 112, 64, device=dev).to(torch.float16)
    row("maxpool 3x3 / 2 (NHWC)", [128, 112, 112, 64], xi.numel() * 2 * 1.25, lambda: maxpool_nhwc(xi, 3, 2, 1))
    xa = torch.randn(8192, 7, 7, 512, device=dev).to(torch.float16)
    row("global average pool (NHWC)", [8192, 7, 7, 512], xa.numel() * 2.0, lambda: global_avgpool_nhwc(xa))
    return out


def bench_conv(n=32, h=56, w=56, c=64, cout=64, r=3, stride=1, pad=1, dtype=torch.float16, flush=True, iters=20):
    from ..providers.gpu_conv import conv2d_nhwc
    x = torch.randn(n, h, w, c, device="cuda").to(dtype)
    wt = (torch.randn(cout, r, r, c, device="cuda") / math.sqrt(r * r * c)).to(dtype)
    b = torch.zeros(cout, device="cuda", dtype=dtype)
    ho, wo = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    out = torch.empty(n, ho, wo, cout, device="cuda", dtype=dtype)
    us = time_kernel(lambda: conv2d_nhwc(x, wt, b, None, stride, pad, 1, relu=True, out=out), iters=iters, flush=flush)
    K.check_status()
    hbm, tf, src = _peaks()
    flops = 2.0 * n * ho * wo * cout * r * r * c
    byts = 2.0 * (x.numel() + wt.numel() + out.numel())
    roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e6
    xn, wn = x.permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last), wt.permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
    us_lib = time_kernel(lambda: torch.relu_(torch.nn.functional.conv2d(xn, wn, b, stride, pad)), iters=iters, flush=flush)
    return {"kernel": "conv_igemm", "shape": [n, h, w, c, cout, r, stride], "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
            "roofline_us": round(roof, 2), "frac_of_" + src: round(roof / us, 3), "cudnn_us": round(us_lib, 2)}


def bench_bitlinear(m=128, n=2560, k=2560, flush=True, iters=20):
    from . import bitnet as B
    x = torch.randn(m, k, device="cuda").bfloat16()
    wq = torch.randint(-1, 2, (n, k), device="cuda", dtype=torch.int8)
    packed = B.ternary_pack(wq)
    q, s = B.act_quant_int8(x)
    us = time_kernel(lambda: B.bitlinear_q(q, s, packed, 0.04, None, n, k, torch.bfloat16), iters=iters, flush=flush)
    us_q = time_kernel(lambda: B.act_quant_int8(x), iters=iters, flush=flush)
    K.check_status()
    hbm, tf, src = _peaks()
    byts = n * k / 4.0 + m * k + m * n * 2.0
    wd = wq.to(torch.bfloat16)
    us_lib = time_kernel(lambda: torch.matmul(x, wd.t()), iters=iters, flush=flush)
    return {"kernel": "bitlinear", "m": m, "n": n, "k": k, "us": round(us, 2), "act_quant_us": round(us_q, 2),
            "gbs": round(byts / us / 1e3, 1), "roofline_us": round(byts / (hbm * 1e9) * 1e6, 2),
            "frac_of_" + src: round(byts / (hbm * 1e9) * 1e6 / us, 3), "dequantised_bf16_cublas_us": round(us_lib, 2)}


def bench_fused_elementwise(rows=131072, h=1024, flush=True, iters=20):
    """The one-launch chain kernel on a 4-operator chain (add a row vector, ReLU, multiply by a full tensor, tanh)
    against the same chain as four library kernels; operands larger than L2."""
    hbm, _, src = _peaks()
    x = torch.randn(rows, h, device="cuda").bfloat16()
    bias = torch.randn(h, device="cuda").bfloat16()
    w = torch.randn(rows, h, device="cuda").bfloat16()
    names, operands = ["Add", "Relu", "Mul", "Tanh"], [bias, None, w, None]
    plan = K.fused_elementwise_plan(x, names, operands)
    us = time_kernel(lambda: K.fused_elementwise(x, names, operands, plan), iters=iters, flush=flush)
    us_lib = time_kernel(lambda: torch.tanh(torch.relu(x + bias) * w), iters=iters, flush=flush)
    byts = 3.0 * rows * h * 2
    return {"kernel": "fused_elementwise", "chain": names, "shape": [rows, h], "us": round(us, 2), "gbs": round(byts / us / 1e3, 1),
            "frac_of_" + src: round(byts / (hbm * 1e9) * 1e6 / us, 3), "four_library_kernels_us": round(us_lib, 2)}


def bench_sampling(rows=2048, vocab=50264, flush=True, iters=20):
    """Device sampler (repeat penalty, temperature 0.8, top-k 50, top-p 0.95) on fp32 logits larger than L2, against the
    library's sort-based form of the same pipeline."""
    import numpy as np
    hbm, _, src = _peaks()
    logits = torch.randn(rows, vocab, device="cuda") * 3
    buf = bytearray(rows * K.SAMPLE_RECORD_BYTES)
    for r in range(rows):
        K.pack_sample_params(buf, r, 0.8, 50, 0.95, 1.1, 1234 + r, 16)
    params = torch.frombuffer(buf, dtype=torch.uint8).cuda()
    recent = torch.randint(0, vocab, (rows, 16), device="cuda", dtype=torch.int32)
    counters = torch.zeros(rows, dtype=torch.int64, device="cuda")
    work = logits.clone()

    def ours():
        work.copy_(logits)                      # the penalty is applied in place
        K.sample(work, params, recent, counters)

    def library():
        z = logits / 0.8
        v, idx = torch.topk(z, 50, dim=-1)
        p = torch.softmax(v, dim=-1)
        keep = (p.cumsum(-1) - p) <= 0.95
        p = p * keep
        return idx.gather(-1, torch.multinomial(p / p.sum(-1, keepdim=True), 1))

    us_copy = time_kernel(lambda: work.copy_(logits), iters=iters, flush=flush)
    us = time_kernel(ours, iters=iters, flush=flush) - us_copy
    us_lib = time_kernel(library, iters=iters, flush=flush)
    K.check_status()
    byts = float(rows) * vocab * 4               # one pass is the floor; the kernel makes several (L2 / L1 resident rows)
    return {"kernel": "sample", "shape": [rows, vocab], "us": round(us, 2), "one_pass_gbs": round(byts / us / 1e3, 1),
            "one_pass_frac_of_" + src: round(byts / (hbm * 1e9) * 1e6 / us, 3), "library_topk_multinomial_us": round(us_lib, 2)}


def resnet_convs():
    shapes = [(32, 224, 224, 8, 64, 7, 2, 3), (32, 56, 56, 64, 64, 3, 1, 1), (32, 56, 56, 64, 128, 3, 2, 1), (32, 28, 28, 128, 128, 3, 1, 1),
              (32, 28, 28, 128, 256, 3, 2, 1), (32, 14, 14, 256, 256, 3, 1, 1), (32, 14, 14, 256, 512, 3, 2, 1), (32, 7, 7, 512, 512, 3, 1, 1),
              (32, 56, 56, 64, 128, 1, 2, 0)]
    return [bench_conv(*s) for s in shapes]


def decode_shapes(batch=256, ctx=416):
    out = []
    for (n, k) in [(3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096), (50257 // 8 * 8 + 8, 1024)]:
        out.append(bench_gemm(batch, n, k))
    out.append(bench_attention(batch, ctx, 16, 64))
    out.append(bench_norm(batch, 1024))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attention", "norm", "decode-shapes", "prefill-shapes", "dense-attention", "fused-single-rank", "memory-kernels", "conv", "resnet-convs", "bitlinear", "bitnet-shapes", "fused-elementwise", "sampling"])
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=416)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ragged", action="store_true", help="attention: context lengths spread around --ctx")
    ap.add_argument("--splits", type=int, default=0, help="attention: CTAs per (row, head); 0 = the default rule")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--causal", action="store_true")
    a = ap.parse_args()
    fl = not a.no_flush
    if a.what == "gemm":
        res = [bench_gemm(a.m, a.n, a.k, bn=a.bn, flush=fl, iters=a.iters)]
    elif a.what == "attention":
        res = [bench_attention(a.batch, a.ctx, a.heads, a.dim, flush=fl, iters=a.iters, ragged=a.ragged,
                               splits=a.splits or None)]
    elif a.what == "memory-kernels":
        res = bench_memory_kernels(flush=fl)
    elif a.what == "norm":
        res = [bench_norm(a.batch, a.n, flush=fl)]
    elif a.what == "conv":
        res = [bench_conv(iters=a.iters, flush=fl)]
    elif a.what == "resnet-convs":
        res = resnet_convs()
    elif a.what == "bitlinear":
        res = [bench_bitlinear(a.m if a.m != 256 else 128, a.n if a.n != 1024 else 2560, a.k if a.k != 1024 else 2560, flush=fl, iters=a.iters)]
    elif a.what == "fused-elementwise":
        res = [bench_fused_elementwise(flush=fl, iters=a.iters)]
    elif a.what == "sampling":
        res = [bench_sampling(flush=fl, iters=a.iters)]
    elif a.what == "bitnet-shapes":
        res = [bench_bitlinear(128, n, k) for (n, k) in [(7680, 2560), (2560, 2560), (13824, 2560), (2560, 6912), (960, 2560), (2560, 864)]]
    elif a.what == "dense-attention":
        # without --batch / --ctx / --heads: the DistilBERT encoder shape (64 x 128 tokens, 12 heads)
        given = lambda flag: any(x == flag or x.startswith(flag + "=") for x in sys.argv)
        res = [bench_dense_attention(a.batch if given("--batch") else 64, a.ctx if given("--ctx") else 128,
                                     a.heads if given("--heads") else 12, a.dim, causal=a.causal, iters=a.iters, flush=fl)]
    elif a.what == "fused-single-rank":
        res = [bench_fused_single_rank(a.m, a.n, a.k, iters=a.iters, flush=fl)]
    elif a.what == "prefill-shapes":
        res = [bench_gemm(8192, n, k) for (n, k) in [(3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096)]]
        res += [bench_gemm(8192, 8192, 8192, iters=5)]
    else:
        res = decode_shapes(a.batch, a.ctx)
    for r in res:
        print(json.dumps(r))


if __name__ == "__main__":
    main()

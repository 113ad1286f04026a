"""Library twins of the hand-written kernels: the same operator shapes timed through cuBLAS / cuDNN / SDPA / NCCL.

    python baseline/library_twins.py gemm | attention-decode | attention-prefill | conv | norm | memory-kernels | bitlinear
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 baseline/library_twins.py gemm-allreduce

Nothing here is on a product path; the numbers are the comparison column of the results tables.  Timing follows the
kernel micro-benchmarks (`ronn_b200/ops/microbench.py`): CUDA events, warm-up, L2 flushed between iterations, median.
The whole-model library baselines are `python bench.py --impl baseline` (decode engine on cuBLAS + SDPA + NCCL) and the
`torch_*` rows printed by `python -m ronn_b200.bench_models resnet18 | distilbert`.
"""
import json
import math
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

_FLUSH = None


def timed(fn, iters=20, warmup=5):
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _FLUSH.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return round(ts[len(ts) // 2], 2)


def gemm():
    out = []
    for (m, n, k) in [(256, 3072, 1024), (256, 1024, 4096), (256, 50264, 1024), (8192, 2304, 768), (8192, 8192, 8192)]:
        a = torch.randn(m, k, device="cuda").bfloat16()
        w = torch.randn(n, k, device="cuda").bfloat16()
        us = timed(lambda: torch.matmul(a, w.t()))
        out.append({"op": "cublas_gemm", "m": m, "n": n, "k": k, "us": us, "tflops": round(2.0 * m * n * k / us / 1e6, 1)})
    return out


def attention_decode(batch=256, ctx=416, heads=16, d=64):
    q = torch.randn(batch, heads, 1, d, device="cuda").bfloat16()
    k = torch.randn(batch, heads, ctx, d, device="cuda").bfloat16()
    v = torch.randn(batch, heads, ctx, d, device="cuda").bfloat16()
    us = timed(lambda: F.scaled_dot_product_attention(q, k, v))
    return [{"op": "sdpa_decode_dense_kv", "batch": batch, "ctx": ctx, "us": us,
             "note": "KV already gathered into a dense tensor; the paged gather is extra"}]


def attention_prefill():
    out = []
    for (b, s, h, d, causal) in [(64, 128, 12, 64, False), (8, 1024, 16, 64, True)]:
        q, k, v = (torch.randn(b, h, s, d, device="cuda").bfloat16() for _ in range(3))
        us = timed(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=causal))
        out.append({"op": "sdpa_prefill", "batch": b, "seq": s, "heads": h, "causal": causal, "us": us})
    return out


def conv():
    out = []
    shapes = [(32, 3, 224, 64, 7, 2, 3), (32, 64, 56, 64, 3, 1, 1), (32, 128, 28, 128, 3, 1, 1), (32, 256, 14, 256, 3, 1, 1),
              (32, 512, 7, 512, 3, 1, 1)]
    for (n, c, hw, co, r, s, p) in shapes:
        x = torch.randn(n, c, hw, hw, device="cuda").half().contiguous(memory_format=torch.channels_last)
        w = torch.randn(co, c, r, r, device="cuda").half().contiguous(memory_format=torch.channels_last)
        b = torch.zeros(co, device="cuda").half()
        us = timed(lambda: torch.relu_(F.conv2d(x, w, b, s, p)))
        out.append({"op": "cudnn_conv_relu", "shape": [n, c, hw, co, r, s], "us": us})
    return out


def norm():
    x = torch.randn(256, 1024, device="cuda").bfloat16()
    g = torch.ones(1024, device="cuda").bfloat16()
    return [{"op": "torch_layer_norm", "rows": 256, "h": 1024, "us": timed(lambda: F.layer_norm(x, (1024,), g, g))}]


def memory_kernels():
    """PyTorch operators on the shapes of `python -m ronn_b200.ops.microbench memory-kernels` (operands larger than L2)."""
    dev, bf = "cuda", torch.bfloat16
    R, H = 131072, 1024
    x, r = torch.randn(R, H, device=dev).to(bf), torch.randn(R, H, device=dev).to(bf)
    g, b = torch.ones(H, device=dev, dtype=bf), torch.zeros(H, device=dev, dtype=bf)
    out = []

    def row(name, shape, byts, fn):
        us = timed(fn)
        out.append({"op": name, "shape": shape, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1)})

    row("torch_layer_norm", [R, H], 2.0 * R * H * 2, lambda: F.layer_norm(x, (H,), g, b))
    row("torch_add+layer_norm", [R, H], 4.0 * R * H * 2, lambda: F.layer_norm(x + r, (H,), g, b))
    row("torch_rms_norm", [R, H], 2.0 * R * H * 2, lambda: F.rms_norm(x, (H,), g, 1e-6))
    row("torch_softmax", [R, H], 2.0 * R * H * 2, lambda: torch.softmax(x, -1))
    row("torch_gelu_tanh", [R, H], 2.0 * R * H * 2, lambda: F.gelu(x, approximate="tanh"))
    row("torch_relu", [R, H], 2.0 * R * H * 2, lambda: torch.relu(x))
    row("torch_add", [R, H], 3.0 * R * H * 2, lambda: x + r)
    row("torch_silu*mul", [R, H], 1.5 * R * H * 2, lambda: F.silu(x[:, :H // 2]) * x[:, H // 2:])
    row("torch_cast_bf16_fp32", [R, H], 3.0 * R * H * 2, lambda: x.float())
    V = 50264
    table = torch.randn(V, H, device=dev).to(bf)
    ids = torch.randint(0, V, (R,), device=dev)
    row("torch_embedding", [R, H], 2.0 * R * H * 2, lambda: F.embedding(ids, table))
    logits = torch.randn(2048, V, device=dev).to(bf)
    row("torch_argmax", [2048, V], 2048.0 * V * 2, lambda: logits.argmax(-1))
    xi = torch.randn(128, 64, 112, 112, device=dev).to(torch.float16).contiguous(memory_format=torch.channels_last)
    row("cudnn_maxpool_3x3_s2", [128, 112, 112, 64], xi.numel() * 2 * 1.25, lambda: F.max_pool2d(xi, 3, 2, 1))
    xa = torch.randn(8192, 512, 7, 7, device=dev).to(torch.float16).contiguous(memory_format=torch.channels_last)
    row("torch_global_avgpool", [8192, 7, 7, 512], xa.numel() * 2.0, lambda: xa.mean(dim=(2, 3)))
    return out


def bitlinear(m=128, n=2560, k=2560):
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randint(-1, 2, (n, k), device="cuda").bfloat16()
    return [{"op": "dequantised_bf16_gemm", "m": m, "n": n, "k": k, "us": timed(lambda: torch.matmul(x, w.t()))}]


def gemm_allreduce():
    import torch.distributed as dist
    from ronn_b200.parallel.group import init_distributed
    rank, world, local = init_distributed("nccl", timeout_s=120)
    out = []
    for (m, n, k) in [(256, 1024, 1024), (256, 1024, 4096), (8192, 1024, 4096)]:
        a = torch.randn(m, k // world, device="cuda").bfloat16()
        w = torch.randn(n, k // world, device="cuda").bfloat16()

        def call():
            y = torch.matmul(a, w.t())
            dist.all_reduce(y)
        us = timed(call)
        t = torch.tensor([us], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.append({"op": "cublas_gemm+nccl_allreduce", "m": m, "n": n, "k_local": k // world, "world": world,
                    "us": round(t.item(), 2)})
    if rank == 0:
        for r in out:
            print(json.dumps(r))
    sys.stdout.flush()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    fns = {"gemm": gemm, "attention-decode": attention_decode, "attention-prefill": attention_prefill, "conv": conv,
           "norm": norm, "memory-kernels": memory_kernels, "bitlinear": bitlinear, "gemm-allreduce": gemm_allreduce}
    if what not in fns:
        sys.exit(f"unknown twin '{what}'; one of {sorted(fns)}")
    res = fns[what]()
    for r in res or []:
        print(json.dumps(r))

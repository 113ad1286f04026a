"""Model-level latency / throughput benchmarks through the public API (Model -> create_session -> run).

    python -m ronn_b200.bench_models resnet18  [--batch 32] [--iters 50]     p50 latency, fp16, O3, GPU provider
    python -m ronn_b200.bench_models mlp784    [--iters 2000]                p50 latency, f32, CPU provider
    python -m ronn_b200.bench_models distilbert [--batch 64 --seq 128]       p50 latency / sequences per second, bf16
    python -m ronn_b200.bench_models bitnet [--batch 128]                    BitNet 2B-style decode tokens/s (TP under torchrun)

Each benchmark also times a plain PyTorch library implementation of the same network on the same box
(cuDNN / cuBLAS / SDPA) as the comparison baseline.  Timing: CUDA events around ``session.run`` with the input
already on the device, after warm-up; the L2 is flushed between iterations by writing a 256 MB buffer.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time

import torch


def _p50_cuda(fn, iters, warmup=5, flush=True):
    buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts), min(ts)


def bench_resnet18(batch=32, iters=50, image=224):
    import torch.nn as nn
    from . import Model, SessionOptions
    from .models.resnet18 import build_resnet18
    graph = build_resnet18(dtype=torch.float16, seed=0)
    model = Model.from_graph(graph)
    x = torch.randn(batch, 3, image, image, device="cuda", dtype=torch.float16)
    out = {}
    for name, graphed in (("ours_cuda_graph", True), ("ours_eager", False)):
        sess = model.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3")
                                    .with_dtype("fp16").with_cuda_graph(graphed))
        p50, best = _p50_cuda(lambda: sess.run({"input": x}), iters)
        out[name] = {"p50_ms": round(p50, 4), "min_ms": round(best, 4), "images_per_s": round(batch / p50 * 1e3, 1)}
        logits = sess.run({"input": x})["logits"].float()
    from .ops import kernels as K
    K.check_status()
    # library baseline: same weights in a torch module, fp16 channels_last, cuDNN
    init = graph.initializers

    class Block(nn.Module):
        def __init__(self, prefix, cin, cout, stride):
            super().__init__()
            self.a = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
            self.bna = nn.BatchNorm2d(cout)
            self.b = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
            self.bnb = nn.BatchNorm2d(cout)
            self.down = None
            if stride != 1 or cin != cout:
                self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False), nn.BatchNorm2d(cout))
            self.a.weight.data = init[f"{prefix}.a.weight"].clone()
            self.b.weight.data = init[f"{prefix}.b.weight"].clone()
            if self.down is not None:
                self.down[0].weight.data = init[f"{prefix}.down.weight"].clone()

        def forward(self, x):
            y = torch.relu(self.bna(self.a(x)))
            y = self.bnb(self.b(y))
            return torch.relu(y + (x if self.down is None else self.down(x)))

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = nn.Conv2d(3, 64, 7, 2, 3, bias=False)
            self.stem.weight.data = init["stem.weight"].clone()
            self.bn = nn.BatchNorm2d(64)
            blocks, cin = [], 64
            for stage, cout in enumerate((64, 128, 256, 512)):
                for blk in range(2):
                    blocks.append(Block(f"layer{stage + 1}.{blk}", cin, cout, 2 if (stage > 0 and blk == 0) else 1))
                    cin = cout
            self.blocks = nn.Sequential(*blocks)
            self.fc = nn.Linear(512, 1000)
            self.fc.weight.data = init["fc.weight"].clone()
            self.fc.bias.data = init["fc.bias"].clone()

        def forward(self, x):
            x = torch.max_pool2d(torch.relu(self.bn(self.stem(x))), 3, 2, 1)
            x = self.blocks(x)
            return self.fc(x.mean((2, 3)))

    net = Net().cuda().half().eval().to(memory_format=torch.channels_last)
    xc = x.to(memory_format=torch.channels_last)
    with torch.no_grad():
        p50, best = _p50_cuda(lambda: net(xc), iters)
        out["torch_cudnn_eager"] = {"p50_ms": round(p50, 4), "min_ms": round(best, 4)}
        ref = net(xc).float()
        g = torch.cuda.CUDAGraph()
        static = xc.clone()
        for _ in range(3):
            net(static)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            y = net(static)
        p50, best = _p50_cuda(lambda: g.replay(), iters)
        out["torch_cudnn_cuda_graph"] = {"p50_ms": round(p50, 4), "min_ms": round(best, 4)}
    rel = float((logits - ref).abs().max() / ref.abs().max())
    flops = 2 * 1.82e9 * batch
    out["config"] = {"model": "resnet18", "batch": batch, "dtype": "fp16", "layout": "NCHW input, NHWC inside",
                     "max_rel_err_vs_torch": round(rel, 5),
                     "tflops_at_p50": round(flops / (out["ours_cuda_graph"]["p50_ms"] * 1e-3) / 1e12, 1)}
    return out


def bench_mlp784(iters=2000):
    from . import Model, SessionOptions
    from .models.mlp784 import build_mlp784
    graph = build_mlp784()
    model = Model.from_graph(graph)
    x = torch.rand(1, 784)
    out = {}
    for lvl in ("O0", "O3"):
        sess = model.create_session(SessionOptions().with_optimization_level(lvl))
        for _ in range(200):
            sess.run({"input": x})
        ts = []
        for _ in range(iters):
            t = time.perf_counter()
            sess.run({"input": x})
            ts.append((time.perf_counter() - t) * 1e6)
        out[f"ours_cpu_{lvl}"] = {"p50_us": round(statistics.median(ts), 2), "p95_us": round(sorted(ts)[int(0.95 * len(ts))], 2)}
    w1, w2 = graph.initializers["fc1.weight"], graph.initializers["fc2.weight"]
    b1, b2 = graph.initializers["fc1.bias"], graph.initializers["fc2.bias"]
    with torch.no_grad():
        f = lambda: torch.softmax(torch.relu(x @ w1 + b1) @ w2 + b2, -1)
        for _ in range(200):
            f()
        ts = []
        for _ in range(iters):
            t = time.perf_counter()
            f()
            ts.append((time.perf_counter() - t) * 1e6)
    out["torch_cpu_eager"] = {"p50_us": round(statistics.median(ts), 2)}
    out["config"] = {"model": "mlp 784-128-10", "batch": 1, "dtype": "f32", "reference_target": "P50 < 10 ms"}
    return out


def bench_distilbert(batch=64, seq=128, iters=20):
    """Encoder forward, batch x seq tokens.  Under ``torchrun`` the runner is tensor parallel over all ranks (fused
    GEMM + all-reduce + LayerNorm kernels) and the time is the maximum over ranks; on one GPU the graph session and a
    PyTorch library implementation (cuBLAS + SDPA) are timed as well."""
    import os
    from . import Model, SessionOptions
    from .models.distilbert import build_distilbert
    from .serving.encoder_runner import EncoderRunner
    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = None
    if world > 1:
        from .parallel import make_comm
        from .parallel.group import init_distributed
        rank, world, local = init_distributed()
        torch.cuda.set_device(local)
        comm = make_comm(os.environ.get("RONN_TP_COMM", "fused"), torch.device("cuda", local))
    else:
        rank = 0
    graph = build_distilbert(dtype=torch.bfloat16, seed=0)
    model = Model.from_graph(graph)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 30522, (batch, seq), generator=gen).cuda()
    mask = torch.ones(batch, seq, dtype=torch.int64, device="cuda")
    out = {}
    sp = world > 1 and os.environ.get("RONN_ENCODER_SP", "0") == "1"      # token-sharded layout on the fused kernels
    runner = EncoderRunner(graph, dtype=torch.bfloat16, comm=comm, sequence_parallel=sp)
    static_ids = ids.clone()
    runner.forward(static_ids, mask)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = runner.forward(static_ids, mask)
    p50, best = _p50_cuda(g.replay, iters)
    if comm is not None:
        p50 = comm.max_over_ranks(p50)
    out["runner_cuda_graph"] = {"p50_ms": round(p50, 4), "sequences_per_s": round(batch / p50 * 1e3, 1)}
    runner.ops.check()
    if world == 1:
        for name, graphed in (("session_cuda_graph", True), ("session_eager", False)):
            sess = model.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3")
                                        .with_dtype("bf16").with_cuda_graph(graphed))
            p50, best = _p50_cuda(lambda: sess.run({"input_ids": ids, "attention_mask": mask}), iters)
            out[name] = {"p50_ms": round(p50, 4), "sequences_per_s": round(batch / p50 * 1e3, 1)}
        lib = EncoderRunner(graph, dtype=torch.bfloat16, backend="torch")
        ref = lib.forward(ids, mask)
        p50, best = _p50_cuda(lambda: lib.forward(ids, mask), iters)
        out["torch_ops_eager"] = {"p50_ms": round(p50, 4)}
        out["max_abs_err_vs_torch_ops"] = round((y.float() - ref.float()).abs().max().item(), 4)
    out["config"] = {"model": "distilbert-base", "batch": batch, "seq": seq, "dtype": "bf16", "tp": world,
                     "sequence_parallel": bool(sp), "l2": "flushed between iterations"}
    if world > 1:
        import sys
        if rank == 0:
            print(json.dumps(out))
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)
    return out


def bench_bitnet(batch=128, steps=32, warmup=3, prompt=64, layers=24, comm=None, standalone=True):
    """BitNet b1.58 2B-style decoder (24 layers, hidden 2560, 20 heads, FFN 6912, vocab 32000; random ternary weights
    packed 2-bit, int8 activations), decode tokens/s at a fixed batch through the serving engine (paged KV,
    CUDA-graph decode).  Under ``torchrun`` the model is tensor parallel over all ranks; the time is the maximum over
    ranks, measured with CUDA events around whole engine steps."""
    import os
    import sys
    import numpy as np
    from . import Model
    from .models.bitnet_llama import BitNetConfig, build_bitnet_llama
    from .serving import EngineConfig, LLMEngine, SamplingParams
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local = 0, 0
    if world > 1:
        from .parallel import make_comm
        from .parallel.group import init_distributed
        rank, world, local = init_distributed()
        torch.cuda.set_device(local)
        if comm is None:                     # a caller that already owns a communicator passes it in
            comm = make_comm(os.environ.get("RONN_TP_COMM", "fused"), torch.device("cuda", local))
    dev = torch.device("cuda", local)
    cfg = BitNetConfig(n_layer=layers)
    model = Model.from_graph(build_bitnet_llama(cfg, dtype=torch.bfloat16, seed=0, with_lm_head=False))
    new_tokens = steps + warmup + 4
    ecfg = EngineConfig(max_num_seqs=batch, max_batch_tokens=8192, max_model_len=1024, dtype="bf16", backend="kernels",
                        use_cuda_graph=True, tp_size=world, tp_comm=os.environ.get("RONN_TP_COMM", "fused"),
                        num_blocks=batch * 16)
    eng = LLMEngine(model, ecfg, device=dev, comm=comm)
    rng = np.random.default_rng(7)
    for _ in range(batch):
        eng.add_request(rng.integers(0, cfg.vocab_size, size=prompt).tolist(), SamplingParams(max_new_tokens=new_tokens))
    while eng.sched.num_waiting > 0:
        eng.step()
    for _ in range(max(warmup, 3)):
        eng.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        torch.distributed.barrier()
    e0.record()
    for _ in range(steps):
        out = eng.step()
        assert len(out) == batch
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if comm is not None:
        ms = comm.max_over_ranks(ms)
    res = {"decode_tokens_per_s": round(batch * steps / ms * 1e3, 1), "ms_per_step": round(ms / steps, 4),
           "config": {"model": "bitnet-b1.58-2b-style" if layers == 24 else f"bitnet-{layers}L", "batch": batch,
                      "prompt": prompt, "steps": steps, "dtype": "ternary 2-bit x int8 (bf16 elsewhere)", "tp": world,
                      "l2": "KV + packed weights per step exceed L2"}}
    if world > 1 and standalone:
        if rank == 0:
            print(json.dumps(res))
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)
    return res


def resnet18_latency(batch=32, iters=30, image=224):
    """ResNet-18, fp16, NCHW input [batch, 3, image, image], O3 (Conv + BN + ReLU fused, NHWC inside), GPU provider with
    CUDA-graph replay, through Model -> create_session -> run.  Returns the p50 latency with the input already on the
    device and the p50 of the whole call a user makes: input copied from pinned host memory, run, logits copied back."""
    from . import Model, SessionOptions
    from .models.resnet18 import build_resnet18
    model = Model.from_graph(build_resnet18(dtype=torch.float16, seed=0))
    sess = model.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3")
                                .with_dtype("fp16").with_cuda_graph(True))
    x_host = torch.randn(batch, 3, image, image, dtype=torch.float16).pin_memory()
    x = x_host.cuda()
    p50, best = _p50_cuda(lambda: sess.run({"input": x}), iters)
    logits_host = torch.empty((batch, 1000), dtype=torch.float16).pin_memory()

    def end_to_end():
        xd = x_host.to("cuda", non_blocking=True)
        logits_host.copy_(sess.run({"input": xd})["logits"], non_blocking=True)

    e2e, _ = _p50_cuda(end_to_end, iters)
    from .ops import kernels as K
    K.check_status()
    return {"p50_ms": round(p50, 4), "min_ms": round(best, 4), "e2e_p50_ms": round(e2e, 4),
            "images_per_s": round(batch / p50 * 1e3, 1), "h2d_bytes": x_host.numel() * 2, "d2h_bytes": logits_host.numel() * 2,
            "config": "fp16 NCHW [%d,3,%d,%d], O3, CUDA graph, L2 flushed between runs" % (batch, image, image)}


def bench_serving(concurrency=(1, 4, 16, 32), prompt=128, new_tokens=64, model="gpt2-medium", device=None):
    """Closed-loop serving at fixed concurrency: `c` requests in flight (each replaced when it finishes, 3 c requests in
    all), reporting tokens/s and the TTFT / inter-token-latency percentiles of the continuous-batching design's test
    plan (docs/new/RONN-Continuous-Batching-Branch-Prompt.md:442-470).  On a CUDA device the engine uses the kernel
    backend in bf16; on CPU the PyTorch backend in fp32 (use a tiny model there)."""
    from . import Model
    from .models.gpt2 import GPT2Config, build_gpt2
    from .serving import EngineConfig, LLMEngine, SamplingParams
    cuda = torch.cuda.is_available() if device is None else torch.device(device).type == "cuda"
    dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
    cfg = GPT2Config.medium() if model == "gpt2-medium" else GPT2Config.tiny()
    graph = build_gpt2(cfg, dtype=torch.bfloat16 if cuda else torch.float32)
    m = Model.from_graph(graph)
    out = []
    g = torch.Generator().manual_seed(0)
    for c in concurrency:
        max_len = prompt + new_tokens + 16
        blocks = (c + 1) * (-(-max_len // 16)) + 8          # sized for the run, not for the whole device memory
        eng = LLMEngine(m, EngineConfig(max_num_seqs=max(c, 1), max_batch_tokens=max(2048, prompt * 4),
                                        max_model_len=max_len, num_blocks=blocks, dtype="bf16" if cuda else "fp32",
                                        backend="kernels" if cuda else "torch"), device=dev)
        total = 3 * c
        make = lambda: torch.randint(0, cfg.vocab_size, (prompt,), generator=g).tolist()
        eng.generate([make()], SamplingParams(max_new_tokens=4))                    # warm-up: graphs, workspaces
        eng.metrics.ttft.clear()
        eng.metrics.itl.clear()
        submitted = 0
        live = set()
        t0 = time.perf_counter()
        generated = 0
        while submitted < total or live:
            while submitted < total and len(live) < c:
                live.add(eng.add_request(make(), SamplingParams(max_new_tokens=new_tokens)))
                submitted += 1
            eng.step()
            for rid in [r for r in live if eng.requests[r].finished]:
                generated += len(eng.requests[rid].output_tokens)
                live.discard(rid)
        wall = time.perf_counter() - t0
        d = eng.metrics.as_dict()
        out.append({"concurrency": c, "requests": total, "tokens_per_s": round(generated / wall, 1),
                    "ttft_ms": {k: round(d[f"ttft_{k}"] * 1e3, 2) for k in ("p50", "p95", "p99")},
                    "itl_ms": {k: round(d[f"itl_{k}"] * 1e3, 3) for k in ("p50", "p95", "p99")}})
        del eng                                             # the next engine allocates its own cache
        if cuda:
            torch.cuda.empty_cache()
    return {"model": model, "prompt": prompt, "new_tokens": new_tokens, "device": str(dev), "results": out}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["resnet18", "mlp784", "distilbert", "bitnet", "serving"])
    ap.add_argument("--model", default="gpt2-medium", choices=["gpt2-medium", "gpt2-tiny"])
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--iters", type=int, default=0)
    a = ap.parse_args()
    if a.what == "resnet18":
        res = bench_resnet18(a.batch or 32, a.iters or 50)
    elif a.what == "mlp784":
        res = bench_mlp784(a.iters or 2000)
    elif a.what == "serving":
        res = bench_serving(model=a.model, prompt=a.seq, new_tokens=a.iters or 64)
    elif a.what == "bitnet":
        res = bench_bitnet(a.batch or 128, a.iters or 32, layers=a.layers)
    else:
        res = bench_distilbert(a.batch or 64, a.seq, a.iters or 20)
    print(json.dumps(res))


if __name__ == "__main__":
    main()

"""Library arm of the headline benchmark: GPT-2-medium decode on PyTorch operators only.

Same model (random-init GPT-2 medium, bf16), same workload (256 sequences, prompts U(64,512), the timed window is K
consecutive decode steps centred on token 128 of 256) and the same tensor-parallel layout as ``bench.py``, but every
operator is a library call: cuBLAS (``F.linear``), ``F.scaled_dot_product_attention`` over a contiguous per-sequence
KV cache [batch, heads, max_len, head_dim] with a length mask, ``F.layer_norm``, ``F.gelu``, NCCL all-reduce for the
row-parallel projections and an NCCL all-gather for the sharded argmax.  One decode step is captured once as a CUDA
graph (the KV window is the longest context of the timed window rounded up to 64) and replayed, so the arm pays no
Python or launch overhead that the product path does not pay.  Nothing of ``ronn_b200``'s kernels or engine runs here;
the package is only used to build the same random weights.

    python bench.py --impl baseline --gpus N --steps K --warmup W        (N > 1 under torch.distributed.run)
"""
from __future__ import annotations

import math
import time

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchGPT2Decoder:
    def __init__(self, init, cfg, device, rank: int, world: int, batch: int, max_len: int):
        H, nh = cfg.n_embd, cfg.n_head
        assert nh % world == 0, "the library arm shards whole heads evenly"
        self.cfg, self.dev, self.rank, self.world, self.B, self.max_len = cfg, device, rank, world, batch, max_len
        self.d = H // nh
        self.nh_local = nh // world
        hs, hn = rank * self.nh_local * self.d, self.nh_local * self.d
        ffn_local = 4 * H // world
        f0 = rank * ffn_local
        to = lambda t: t.to(device, torch.bfloat16).contiguous()
        self.wte, self.wpe = to(init["wte"]), to(init["wpe"])
        self.lnf = (to(init["ln_f.weight"]), to(init["ln_f.bias"]))
        self.layers = []
        for i in range(cfg.n_layer):
            p = f"h.{i}"
            wqkv, bqkv = init[f"{p}.attn.c_attn.weight"], init[f"{p}.attn.c_attn.bias"]
            cols = torch.cat([torch.arange(hs, hs + hn), H + torch.arange(hs, hs + hn), 2 * H + torch.arange(hs, hs + hn)])
            self.layers.append(dict(
                ln1=(to(init[f"{p}.ln_1.weight"]), to(init[f"{p}.ln_1.bias"])),
                ln2=(to(init[f"{p}.ln_2.weight"]), to(init[f"{p}.ln_2.bias"])),
                wqkv=to(wqkv[:, cols].t()), bqkv=to(bqkv[cols]),
                wo=to(init[f"{p}.attn.c_proj.weight"][hs:hs + hn, :].t()), bo=to(init[f"{p}.attn.c_proj.bias"]),
                wfc=to(init[f"{p}.mlp.c_fc.weight"][:, f0:f0 + ffn_local].t()), bfc=to(init[f"{p}.mlp.c_fc.bias"][f0:f0 + ffn_local]),
                wpr=to(init[f"{p}.mlp.c_proj.weight"][f0:f0 + ffn_local, :].t()), bpr=to(init[f"{p}.mlp.c_proj.bias"])))
        vs = -(-cfg.vocab_size // world)
        self.v0 = min(rank * vs, cfg.vocab_size)
        self.lm_head = self.wte[self.v0: min(self.v0 + vs, cfg.vocab_size)]
        shape = (batch, self.nh_local, max_len, self.d)
        self.k = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(cfg.n_layer)]
        self.v = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(cfg.n_layer)]
        self.rows = torch.arange(batch, device=device)

    def _ar(self, y):
        if self.world > 1:
            dist.all_reduce(y)
        return y

    def _block_tail(self, L, x, att):
        H = self.cfg.n_embd
        x = x + self._ar(F.linear(att, L["wo"])) + L["bo"]
        h = F.layer_norm(x, (H,), *L["ln2"], self.cfg.layer_norm_epsilon if hasattr(self.cfg, "layer_norm_epsilon") else 1e-5)
        f = F.gelu(F.linear(h, L["wfc"], L["bfc"]), approximate="tanh")
        return x + self._ar(F.linear(f, L["wpr"])) + L["bpr"]

    def _token(self, x):
        x = F.layer_norm(x, (self.cfg.n_embd,), *self.lnf, 1e-5)
        logits = F.linear(x, self.lm_head).float()
        mx, idx = logits.max(dim=-1)
        idx = idx + self.v0
        if self.world > 1:
            both = torch.stack([mx, idx.float()], dim=0).contiguous()
            allb = torch.empty((self.world,) + tuple(both.shape), dtype=both.dtype, device=both.device)
            dist.all_gather_into_tensor(allb, both)
            best = allb[:, 0].argmax(dim=0)
            idx = allb[:, 1].gather(0, best[None])[0].long()
        return idx

    @torch.no_grad()
    def prefill(self, prompts):
        """Padded causal prefill, a few sequences at a time (untimed); fills the dense KV cache, returns first tokens."""
        lens = torch.tensor([len(p) for p in prompts], device=self.dev)
        first = torch.zeros(self.B, dtype=torch.long, device=self.dev)
        H = self.cfg.n_embd
        for s0 in range(0, self.B, 32):
            chunk = prompts[s0:s0 + 32]
            Lm = max(len(p) for p in chunk)
            ids = torch.zeros(len(chunk), Lm, dtype=torch.long, device=self.dev)
            for i, p in enumerate(chunk):
                ids[i, :len(p)] = torch.tensor(p, device=self.dev)
            pos = torch.arange(Lm, device=self.dev)
            x = self.wte[ids] + self.wpe[pos][None]
            for li, L in enumerate(self.layers):
                h = F.layer_norm(x, (H,), *L["ln1"], 1e-5)
                qkv = F.linear(h, L["wqkv"], L["bqkv"]).view(len(chunk), Lm, 3, self.nh_local, self.d).permute(2, 0, 3, 1, 4)
                q, k, v = qkv[0], qkv[1], qkv[2]
                self.k[li][s0:s0 + len(chunk), :, :Lm] = k
                self.v[li][s0:s0 + len(chunk), :, :Lm] = v
                att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
                att = att.permute(0, 2, 1, 3).reshape(len(chunk), Lm, self.nh_local * self.d)
                x = self._block_tail(L, x, att)
            last = x[torch.arange(len(chunk), device=self.dev), lens[s0:s0 + len(chunk)] - 1]
            first[s0:s0 + len(chunk)] = self._token(last)
        return first, lens.clone()

    @torch.no_grad()
    def decode_step(self, ids, pos, window: int):
        """ids, pos: [B] device tensors (pos = index the new token is written at).  Returns the next ids."""
        H, B = self.cfg.n_embd, self.B
        x = self.wte[ids] + self.wpe[pos]
        keep = (torch.arange(window, device=self.dev)[None, :] <= pos[:, None])[:, None, None, :]
        for li, L in enumerate(self.layers):
            h = F.layer_norm(x, (H,), *L["ln1"], 1e-5)
            qkv = F.linear(h, L["wqkv"], L["bqkv"]).view(B, 3, self.nh_local, self.d)
            self.k[li][self.rows, :, pos] = qkv[:, 1]
            self.v[li][self.rows, :, pos] = qkv[:, 2]
            att = F.scaled_dot_product_attention(qkv[:, 0].unsqueeze(2), self.k[li][:, :, :window], self.v[li][:, :, :window],
                                                 attn_mask=keep)
            x = self._block_tail(L, x, att.reshape(B, self.nh_local * self.d))
        return self._token(x)


def run(args, rank: int, world: int, local: int, ClockSampler):
    """Runs the library arm and returns the JSON record (on every rank; rank 0 prints it)."""
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    dev = torch.device("cuda", local)
    K, W = args.steps, max(args.warmup, 3)
    cfg = GPT2Config(n_layer=args.layers)
    graph = build_gpt2(cfg, dtype=torch.bfloat16, seed=0, with_lm_head=False)
    rng = np.random.default_rng(1234)
    lens = rng.integers(64, 513, size=args.requests)
    prompts = [rng.integers(0, cfg.vocab_size, size=int(n)).tolist() for n in lens]
    advance = max((args.new_tokens - K) // 2 - W, 0)
    last_pos = int(lens.max()) + advance + W + K + 1
    window = min(-(-last_pos // 64) * 64, 1024)
    model = TorchGPT2Decoder(graph.initializers, cfg, dev, rank, world, args.requests, window)
    t_pf = time.perf_counter()
    ids, pos = model.prefill(prompts)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t_pf
    # static buffers of the captured step
    ids_buf, pos_buf = ids.clone(), pos.clone()
    host_pos = torch.zeros(args.requests, dtype=torch.long).pin_memory()
    host_tok = torch.zeros(args.requests, dtype=torch.long).pin_memory()

    def one():
        nxt = model.decode_step(ids_buf, pos_buf, window)
        ids_buf.copy_(nxt)
        pos_buf.add_(1)
        return nxt

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        one()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = one()
    for _ in range(advance + W - 1):
        g.replay()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    sync_all()
    sampler.start()
    t0 = time.perf_counter()
    cur = pos_buf.cpu()
    for i in range(K):
        # end to end: the step's positions come from pinned host memory, its tokens are read back
        host_pos.copy_(cur + i)
        starts[i].record()
        pos_buf.copy_(host_pos, non_blocking=True)
        g.replay()
        host_tok.copy_(out, non_blocking=True)
        ends[i].record()
        torch.cuda.current_stream().synchronize()
    sync_all()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    dev_ms = sum(a.elapsed_time(b) for a, b in zip(starts, ends))
    if world > 1:
        t = torch.tensor([dev_ms, wall], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, wall = float(t[0]), float(t[1])
    tokens = args.requests * K
    return {
        "metric": "GPT-2 decode tokens/s (continuous batching, paged KV)", "value": round(tokens / (dev_ms / 1e3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "library-baseline",
        "config": {"model": "gpt2-medium" if cfg.n_layer == 24 else f"gpt2-medium-{cfg.n_layer}L",
                   "global_batch": args.requests, "seq_len": "prompts U(64,512) + 256 new tokens",
                   "parallelism": f"tp{world}", "kv": f"contiguous per-sequence cache, SDPA over a {window}-token window with a length mask",
                   "operators": "cuBLAS F.linear, F.scaled_dot_product_attention, F.layer_norm, F.gelu, NCCL all-reduce; one CUDA graph per step",
                   "mean_context_in_window": round(float(np.mean(lens)) + advance + W + K / 2, 1),
                   "l2": "inputs larger than L2 (KV read per step >> 126 MB)", "prefill_seconds_untimed": round(prefill_s, 3)},
        "clocks": clocks,
        "e2e": {"value": round(tokens / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": args.requests * 8,
                "d2h_bytes_per_step": args.requests * 8, "ms_per_step": round(wall * 1e3 / K, 4)},
        "gpu_launches": 0,
    }

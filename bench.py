#!/usr/bin/env python
"""Headline benchmark: GPT-2-medium decode tokens/s under continuous batching.

Workload (fixed by the benchmark definition): GPT-2 medium (24 layers, hidden 1024, 16 heads,
vocab 50257), bf16, paged KV cache with 16-token blocks, 256 concurrent requests with prompt
lengths U(64,512) and 256 generated tokens each, random token ids and random-init weights,
tensor-parallel over N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W          (N>1: launched once per rank by torchrun)

A "step" is one engine iteration that decodes one token for every one of the 256 sequences.
All prompts are prefilled first, the engine is advanced so that the timed window is centred on
the middle of the 256-token generation, W untimed warm-up steps run, then exactly K steps are
timed between barrier + synchronize pairs.  Two numbers come from those same K steps:

  value  device time: CUDA events around each step on the launching stream (from the start of the
         step's input upload to the end of its token read-back), summed, max over ranks
  e2e    wall clock of the K ``engine.step()`` calls (host scheduling, pinned-memory H2D of the
         step inputs, graph replay, D2H of the sampled tokens), max over ranks

Further keys of the line:
  e2e_full          wall-clock tokens/s of a WHOLE run of the workload through ``engine.step()``: 256 requests are
                    admitted, prefilled in chunks, decoded to 256 new tokens each and retired (continuous batching
                    from the first admission to the last finished request)
  gpu_launches      launcher calls of the in-tree sm_100a kernel library inside the timed window, counted by the
                    library's call counter (graph replays add the count recorded at capture)
  resnet18_p50_ms   (N = 1) ResNet-18 fp16 batch 32, O3, p50 latency through Model.create_session / session.run
  bitnet_tp8_tokens_s  (N = 8) BitNet b1.58 2B-style decoder, batch 128 decode, tensor parallel over the 8 GPUs
  vs_baseline       value divided by the library arm's tokens/s at the same N, from the kept logs (the reference
                    publishes no number for this metric)

``--impl baseline`` runs the library arm (``baseline/library_decode.py``: cuBLAS + SDPA + NCCL, one CUDA graph per
step); ``--impl reference`` reports that the reference cannot be built here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def reference_arm():
    if os.environ.get("RANK", "0") != "0":          # launched once per GPU for N > 1: one line, from rank 0
        return 0
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a Rust/Cargo workspace (no setup.py/pyproject at its root, no cargo/"
                                     "rustc/maturin in the image, 12 workspace members missing, gpu feature does not "
                                     "compile); offline pip install fails, nothing to run"}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML inside the process every 25 ms
    (read-only queries; the device is found by the UUID CUDA reports, so CUDA_VISIBLE_DEVICES does not matter), or, when
    NVML cannot be loaded, by running nvidia-smi every 150 ms."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None
        self.source = "nvidia-smi"
        self._nvml = self._handle = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = "GPU-" + str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            try:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._sample_nvml(pynvml)                  # one trial query: any failure falls back to nvidia-smi
            self.samples.clear()
            self._nvml, self.source = pynvml, "nvml"
        except Exception:
            self._nvml = self._handle = None

    def _sample_nvml(self, nv):
        sm = float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        mask = int(get(self._handle))
        bit = lambda *names: next((int(getattr(nv, n)) for n in names if hasattr(nv, n)), 0)
        flags = [
            mask & bit("nvmlClocksEventReasonHwSlowdown", "nvmlClocksThrottleReasonHwSlowdown"),
            mask & bit("nvmlClocksEventReasonHwThermalSlowdown", "nvmlClocksThrottleReasonHwThermalSlowdown"),
            mask & bit("nvmlClocksEventReasonSwThermalSlowdown", "nvmlClocksThrottleReasonSwThermalSlowdown"),
            mask & bit("nvmlClocksEventReasonSwPowerCap", "nvmlClocksThrottleReasonSwPowerCap"),
        ]
        self.samples.append([str(sm), str(self._max), "0"] + ["Active" if f else "Not Active" for f in flags])

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml(self._nvml)
                else:
                    out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                    f = [x.strip() for x in out.strip().split(",")]
                    if len(f) >= 7:
                        self.samples.append(f)
            except Exception:
                pass
            self._stop.wait(0.025 if self._nvml is not None else 0.15)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples), "source": self.source}


# tokens/s of the library arm (`bench.py --impl baseline`) on this pool's B200s, by GPU count; the same numbers and the
# logs they come from are kept under profiles/logs (bench_library_n*.log).  None: not measured at that GPU count.
LIBRARY_BASELINE_TOKENS_S = {1: 51121.5, 2: 62437.2, 4: 78555.7, 8: 71408.2}


def library_baseline_tokens_s(world: int):
    return LIBRARY_BASELINE_TOKENS_S.get(world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--tp-comm", default=os.environ.get("RONN_TP_COMM", "fused"), choices=["fused", "nccl"])
    ap.add_argument("--layers", type=int, default=24, help=argparse.SUPPRESS)       # smoke runs only
    ap.add_argument("--no-extras", action="store_true", help="skip the ResNet-18 (N=1) and BitNet (N=8) side benchmarks")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()

    import numpy as np
    import torch
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.parallel.group import TPComm, init_distributed
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams

    rank, world, local = init_distributed()
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.impl == "baseline":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import library_decode
        rec = library_decode.run(args, rank, world, local, ClockSampler)
        if rank == 0:
            print(json.dumps(rec))
        sys.stdout.flush()
        if world > 1:
            torch.cuda.synchronize()
            os._exit(0)
        return 0
    K, W = args.steps, max(args.warmup, 3)
    new_tokens = max(args.new_tokens, K + W + 2)

    cfg = GPT2Config(n_layer=args.layers)
    graph = build_gpt2(cfg, dtype=torch.bfloat16, seed=0, with_lm_head=False)
    model = Model.from_graph(graph)
    backend = "kernels"
    ecfg = EngineConfig(max_num_seqs=args.requests, max_batch_tokens=8192, max_model_len=1024, dtype="bf16",
                        backend=backend, use_cuda_graph=True, tp_size=world, tp_comm=args.tp_comm,
                        num_blocks=args.requests * 50)
    if world > 1:
        from ronn_b200.parallel import make_comm
        comm = make_comm(ecfg.tp_comm, dev)
    else:
        comm = None
    eng = LLMEngine(model, ecfg, device=dev, comm=comm)
    def sync_all():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- the whole workload once, end to end: admission, chunked prefill, 256 decode steps per request, retirement
    rng_full = np.random.default_rng(4321)
    lens_full = rng_full.integers(64, 513, size=args.requests)
    prompts_full = [rng_full.integers(0, cfg.vocab_size, size=int(n)).tolist() for n in lens_full]
    # untimed pass over prompts of the same lengths with a few new tokens each: loads kernels, sizes buffers and captures the
    # decode graph of the full batch, as a server that has been up for a while would have
    rng_warm = np.random.default_rng(99)         # other token ids: nothing of the timed pass may sit in the prefix cache
    warm = [eng.add_request(rng_warm.integers(0, cfg.vocab_size, size=int(n)).tolist(), SamplingParams(max_new_tokens=4))
            for n in lens_full]
    while eng.has_unfinished():
        eng.step()
    for i in warm:
        eng.release(i)
    sync_all()
    t_full = time.perf_counter()
    full_ids = [eng.add_request(p, SamplingParams(max_new_tokens=args.new_tokens)) for p in prompts_full]
    full_steps = 0
    while eng.has_unfinished():
        eng.step()
        full_steps += 1
    sync_all()
    full_wall = time.perf_counter() - t_full
    full_tokens = sum(len(eng.requests[i].output_tokens) for i in full_ids)
    for i in full_ids:
        eng.release(i)

    rng = np.random.default_rng(1234)
    lens = rng.integers(64, 513, size=args.requests)
    for n in lens:
        eng.add_request(rng.integers(0, cfg.vocab_size, size=int(n)).tolist(), SamplingParams(max_new_tokens=new_tokens))

    # ---- prefill everything, then advance to the window centred on the middle of the generation
    t_pf = time.perf_counter()
    while eng.sched.num_waiting > 0:
        eng.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t_pf
    advance = max((args.new_tokens - K) // 2 - W, 0)
    for _ in range(advance):
        eng.step()
    for _ in range(W):
        eng.step()
    assert eng.sched.num_running == args.requests, "all requests must be decoding in the timed window"

    sampler = ClockSampler(local)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    sync_all()
    sampler.start()
    t0 = time.perf_counter()
    h2d = d2h = launches = 0
    host_dev = host_book = 0.0
    for i in range(K):
        starts[i].record()
        out = eng.step()
        ends[i].record()
        h2d += eng.h2d_bytes_last
        d2h += eng.d2h_bytes_last
        launches += eng.kernel_launches_last
        host_dev += eng.host_seconds_last[0]
        host_book += eng.host_seconds_last[1]
        assert len(out) == args.requests
    sync_all()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    dev_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    if world > 1:
        c = TPComm()
        dev_ms = c.max_over_ranks(dev_ms)
        wall = c.max_over_ranks(wall)
    parts = len(eng._split_rows(eng._bucket(args.requests)) or [None])
    if world > 1:
        c = TPComm()
        full_wall = c.max_over_ranks(full_wall)
    tokens = args.requests * K
    value = tokens / (dev_ms / 1e3)
    e2e = tokens / wall
    mean_ctx = float(np.mean(lens)) + advance + W + K / 2
    extra = {}
    if world == 1 and not args.no_extras:
        from ronn_b200.bench_models import resnet18_latency
        try:
            r18 = resnet18_latency()
            extra["resnet18_p50_ms"] = r18["p50_ms"]
            extra["resnet18"] = r18
        except Exception as e:                       # the headline line must survive a failure of the side benchmark
            extra["resnet18_error"] = str(e)[:200]
    if world == 8 and not args.no_extras:
        from ronn_b200.bench_models import bench_bitnet
        del eng
        torch.cuda.empty_cache()
        try:
            bn = bench_bitnet(comm=comm, standalone=False)
            extra["bitnet_tp8_tokens_s"] = bn["decode_tokens_per_s"]
            extra["bitnet_tp8"] = bn
        except Exception as e:
            extra["bitnet_tp8_error"] = str(e)[:200]
    lib_base = library_baseline_tokens_s(world)
    if rank == 0:
        print(json.dumps({
            "metric": "GPT-2 decode tokens/s (continuous batching, paged KV)", "value": round(value, 1),
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / lib_base, 3) if lib_base else None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": "gpt2-medium" if cfg.n_layer == 24 else f"gpt2-medium-{cfg.n_layer}L",
                       "global_batch": args.requests, "seq_len": "prompts U(64,512) + 256 new tokens",
                       "kv_block": 16, "parallelism": f"tp{world}", "tp_comm": ecfg.tp_comm if world > 1 else "none",
                       "mean_context_in_window": round(mean_ctx, 1),
                       "timed_window": "K consecutive decode steps centred on token 128 of 256",
                       "l2": "inputs larger than L2 (KV read per step >> 126 MB)",
                       "prefill_seconds_untimed": round(prefill_s, 3),
                       "pdl": os.environ.get("RONN_PDL", "1") != "0",
                       "decode_part_batches": parts,
                       "host_ms_per_step": {"schedule_upload_replay_wait": round(host_dev * 1e3 / K, 4),
                                            "commit_bookkeeping": round(host_book * 1e3 / K, 4)}},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d // K,
                    "d2h_bytes_per_step": d2h // K, "ms_per_step": round(wall * 1e3 / K, 4)},
            "e2e_full": {"value": round(full_tokens / full_wall, 1), "unit": "tokens/s", "requests": args.requests,
                         "generated_tokens": int(full_tokens), "engine_steps": full_steps,
                         "wall_seconds": round(full_wall, 4),
                         "what": "admission + chunked prefill + decode + retirement of the whole workload, wall clock"},
            "gpu_launches": int(launches),
            "baseline_on_this_box": {"tokens_per_s": lib_base, "impl": "bench.py --impl baseline (cuBLAS + SDPA + NCCL, CUDA graph)",
                                     "source": "profiles/logs/bench_library_n%d.log" % world},
            **extra,
        }))
    sys.stdout.flush()
    if world > 1:
        # every rank has contributed to the max-over-ranks reductions above; leave without tearing down NCCL and the
        # symmetric-memory mappings (their teardown after graph-captured collectives can block for minutes)
        torch.cuda.synchronize()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())

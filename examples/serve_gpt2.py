"""Continuous batching over a paged KV cache: many requests of different lengths through one engine."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))      # run from a source checkout

import torch

from ronn_b200 import Model
from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams

cuda = torch.cuda.is_available()
cfg = GPT2Config.small() if cuda else GPT2Config.tiny()
model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16 if cuda else torch.float32))
engine = LLMEngine(model, EngineConfig(max_num_seqs=32, max_model_len=min(512, cfg.n_positions), enable_prefix_cache=True))
g = torch.Generator().manual_seed(0)
prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in torch.randint(4, 100, (48,), generator=g)]
outs = engine.generate(prompts, SamplingParams(max_new_tokens=16))
print(len(outs), "completions; first:", outs[0])
print({k: v for k, v in engine.stats().items() if k in ("prefill_steps", "decode_steps", "generated_tokens", "tokens_per_second", "preemptions", "ttft_p50", "itl_p50")})

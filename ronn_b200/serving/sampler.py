"""Token samplers (docs/new/RONN-Llama-Branch-Prompt.md:1011-1116: repeat penalty -> temperature ->
top-k -> top-p -> softmax -> sample; temperature 0 = greedy)."""
from __future__ import annotations

from typing import List

import torch

from .request import Request


def apply_repeat_penalty(logits: torch.Tensor, tokens: List[int], penalty: float) -> torch.Tensor:
    if penalty == 1.0 or not tokens:
        return logits
    idx = torch.tensor(sorted(set(tokens)), device=logits.device, dtype=torch.long)
    vals = logits[idx]
    logits[idx] = torch.where(vals > 0, vals / penalty, vals * penalty)
    return logits


def sample_row(logits: torch.Tensor, r: Request, generator=None) -> int:
    p = r.params
    logits = logits.float().clone()
    logits = apply_repeat_penalty(logits, r.prompt_tokens[-64:] + r.output_tokens, p.repeat_penalty)
    if p.temperature <= 0:
        return int(torch.argmax(logits))
    logits = logits / p.temperature
    if p.top_k and p.top_k < logits.numel():
        kth = torch.topk(logits, p.top_k).values[-1]
        logits = torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)
    probs = torch.softmax(logits, dim=-1)
    if p.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cum = torch.cumsum(sp, dim=0)
        drop = cum - sp > p.top_p
        sp = torch.where(drop, torch.zeros_like(sp), sp)
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
        probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=generator))


def sample_tokens(logits: torch.Tensor, reqs: List[Request], base_seed=None) -> torch.Tensor:
    """One token per row.  A request with a seed draws from a generator seeded by (seed, tokens generated so far);
    with ``base_seed`` (tensor-parallel engines: the same on every rank) requests without a seed do so too, from
    (base_seed, request id), so that replicated engines draw the same tokens."""
    out = []
    for i, r in enumerate(reqs):
        gen = None
        seed = r.params.seed
        if seed is None and base_seed is not None and r.params.temperature > 0:
            seed = (int(base_seed) ^ (r.id * 0x9E3779B1)) & 0x3FFFFFFFFFFFFFFF
        if seed is not None:
            gen = torch.Generator(device=logits.device).manual_seed(seed + len(r.output_tokens))
        out.append(sample_row(logits[i], r, gen))
    return torch.tensor(out, dtype=torch.int32, device=logits.device)

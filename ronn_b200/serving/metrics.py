"""Engine metrics: queue depth, running / waiting, block-pool utilisation, TTFT, inter-token latency,
tokens/s, batch-size histogram; exported as a dict and as Prometheus text
(the /v1/metrics endpoint of docs/new/RONN-Continuous-Batching-Branch-Prompt.md:377-395)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List


def _pct(xs: List[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    k = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[k]


@dataclass
class EngineMetrics:
    requests_added: int = 0
    requests_finished: int = 0
    failed_steps: int = 0
    swapped_blocks: int = 0            # KV blocks copied to or from the host pool by swap preemption
    prefill_steps: int = 0
    decode_steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    busy_seconds: float = 0.0
    waiting: int = 0
    running: int = 0
    free_blocks: int = 0
    total_blocks: int = 0
    ttft: List[float] = field(default_factory=list)
    itl: List[float] = field(default_factory=list)
    batch_hist: Dict[int, int] = field(default_factory=dict)

    def observe_ttft(self, s: float) -> None:
        self.ttft.append(s)

    def observe_step(self, decode, n_items, n_tokens, n_sampled, seconds, waiting, running, free_blocks, total_blocks):
        if decode:
            self.decode_steps += 1
            self.itl.append(seconds)
        else:
            self.prefill_steps += 1
            self.prompt_tokens += n_tokens
        self.generated_tokens += n_sampled
        self.busy_seconds += seconds
        self.waiting, self.running = waiting, running
        self.free_blocks, self.total_blocks = free_blocks, total_blocks
        b = 1
        while b < n_items:
            b *= 2
        self.batch_hist[b] = self.batch_hist.get(b, 0) + 1
        if len(self.itl) > 65536:
            del self.itl[:32768]

    def as_dict(self) -> Dict[str, object]:
        util = 1.0 - self.free_blocks / self.total_blocks if self.total_blocks else 0.0
        return {"requests_added": self.requests_added, "requests_finished": self.requests_finished,
                "failed_steps": self.failed_steps, "swapped_blocks": self.swapped_blocks, "prefill_steps": self.prefill_steps,
                "decode_steps": self.decode_steps, "prompt_tokens": self.prompt_tokens,
                "generated_tokens": self.generated_tokens,
                "tokens_per_second": self.generated_tokens / self.busy_seconds if self.busy_seconds else 0.0,
                "waiting": self.waiting, "running": self.running, "block_utilization": util,
                "ttft_p50": _pct(self.ttft, 0.5), "ttft_p95": _pct(self.ttft, 0.95), "ttft_p99": _pct(self.ttft, 0.99),
                "itl_p50": _pct(self.itl, 0.5), "itl_p95": _pct(self.itl, 0.95), "itl_p99": _pct(self.itl, 0.99),
                "batch_size_histogram": dict(sorted(self.batch_hist.items()))}

    def prometheus(self) -> str:
        d = self.as_dict()
        lines = []
        for k, v in d.items():
            if isinstance(v, dict):
                for b, c in v.items():
                    lines.append(f'ronn_batch_size_bucket{{le="{b}"}} {c}')
            else:
                lines.append(f"ronn_{k} {v}")
        return "\n".join(lines) + "\n"

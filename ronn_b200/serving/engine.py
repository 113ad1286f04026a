"""LLMEngine: iteration-level continuous batching over the paged KV cache.

Loop of one iteration (docs/new/RONN-Continuous-Batching-Branch-Prompt.md:217-248): the native
scheduler picks a prefill batch (admitting waiting requests while blocks and the token budget
allow) or a decode batch (every running sequence, preempting by recompute when blocks run out);
the step plan is flattened into one pinned host buffer, copied to the device in a single
transfer, executed by the decoder runner (decode steps replay a CUDA graph captured per batch
bucket), and the sampled tokens are read back and committed.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Iterable, List, Optional

import numpy as np
import torch

from ..api.errors import SessionError
from .config import EngineConfig
from .metrics import EngineMetrics
from .model_runner import DecoderArch, DecoderRunner, NoComm
from .request import FinishReason, Priority, Request, RequestState, SamplingParams
from .sampler import sample_tokens
from .scheduler import PLAN_DECODE, PLAN_NONE, PLAN_PREFILL, HostBatchBuffers, Scheduler

_BUCKETS = [1, 2, 4, 8, 16, 32, 64, 96, 128, 160, 192, 224, 256, 320, 384, 448, 512, 768, 1024]


class LLMEngine:
    def __init__(self, model, config: Optional[EngineConfig] = None, device=None, comm=None):
        """``model`` is a ``ronn_b200.Model`` (or anything with ``.graph``) holding a decoder architecture."""
        self.cfg = config or EngineConfig()
        graph = model.graph
        self.arch = DecoderArch.from_metadata(graph.metadata)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        if self.device.type == "cpu" and self.cfg.backend == "kernels":
            self.cfg.backend = "torch"
            if self.cfg.dtype != "fp32":
                self.cfg.dtype = "fp32"
        self.comm = comm or NoComm()
        if self.cfg.max_model_len > self.arch.max_pos and self.arch.rope_base == 0:
            self.cfg.max_model_len = self.arch.max_pos
        self.runner = DecoderRunner(self.arch, graph.initializers, self.cfg, self.device, self.comm)
        self.max_blocks = self.runner.max_blocks_per_seq
        self.sched = Scheduler(self.cfg.block_size, self.runner.num_blocks, self.cfg.max_num_seqs,
                               self.cfg.max_batch_tokens, self.cfg.prefill_chunk, self.cfg.policy,
                               self.cfg.enable_prefix_cache, self.max_blocks)
        max_tokens = max(self.cfg.max_batch_tokens, self.cfg.max_num_seqs)
        self.host = HostBatchBuffers(max_tokens, self.cfg.max_num_seqs, self.max_blocks, pin=self.device.type == "cuda")
        self.dev_buf = torch.zeros(self.host.total, dtype=torch.int32, device=self.device)
        self.sampled_dev = torch.zeros(self.cfg.max_num_seqs, dtype=torch.int32, device=self.device)
        self.sampled_host = torch.zeros(self.cfg.max_num_seqs, dtype=torch.int32)
        if self.device.type == "cuda":
            self.sampled_host = self.sampled_host.pin_memory()
        self.requests: Dict[int, Request] = {}
        self._next_id = 0
        self._graphs: Dict[int, tuple] = {}
        self.metrics = EngineMetrics()
        self.use_graph = bool(self.cfg.use_cuda_graph and self.device.type == "cuda")
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.on_token: Optional[Callable[[Request, int], None]] = None

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_tokens: Iterable[int], params: Optional[SamplingParams] = None,
                    priority: Priority = Priority.NORMAL, request_id: Optional[int] = None) -> int:
        toks = [int(t) for t in prompt_tokens]
        if not toks:
            raise SessionError("empty prompt")
        params = params or SamplingParams()
        if len(toks) + params.max_new_tokens > self.cfg.max_model_len:
            raise SessionError(f"prompt ({len(toks)}) + max_new_tokens ({params.max_new_tokens}) exceeds "
                               f"max_model_len ({self.cfg.max_model_len})")
        rid = self._next_id if request_id is None else int(request_id)
        self._next_id = max(self._next_id, rid) + 1
        self.sched.add(rid, toks, params.max_new_tokens, int(priority))
        self.requests[rid] = Request(rid, toks, params, priority)
        self.metrics.requests_added += 1
        return rid

    def cancel(self, request_id: int) -> bool:
        r = self.requests.get(request_id)
        if r is None or r.finished:
            return False
        self.sched.cancel(request_id)
        r.finish_reason = FinishReason.CANCELLED
        r.finished_at = time.perf_counter()
        return True

    def has_unfinished(self) -> bool:
        return self.sched.num_waiting + self.sched.num_running > 0

    # ------------------------------------------------------------------ device views of the step buffers
    def _dev_field(self, name: str, n: int) -> torch.Tensor:
        off, _ = self.host.offsets[name]
        return self.dev_buf[off:off + n]

    def _batch_views(self, n_tokens: int, n_items: int) -> Dict[str, torch.Tensor]:
        f = self._dev_field
        b = {"token_ids": f("token_ids", n_tokens), "positions": f("positions", n_tokens),
             "slot_mapping": f("slot_mapping", n_tokens), "token_item": f("token_item", n_tokens),
             "ctx_per_token": f("ctx_per_token", n_tokens), "seq_lens": f("seq_lens", n_items),
             "sample_index_clamped": f("sample_index", n_items),
             "block_tables": f("block_tables", n_items * self.max_blocks).view(n_items, self.max_blocks)}
        return b

    def _upload(self, n_tokens: int, n_items: int) -> None:
        """One host-to-device copy of the whole staging region actually used by this step."""
        off_bt, _ = self.host.offsets["block_tables"]
        used = off_bt + n_items * self.max_blocks
        self.dev_buf[:used].copy_(self.host.host[:used], non_blocking=True)
        self.h2d_bytes_last = used * 4

    # ------------------------------------------------------------------ one iteration
    def step(self) -> List[Request]:
        """Run one scheduling iteration.  Returns the requests that produced a token in it."""
        kind = self.sched.schedule()
        if kind == PLAN_NONE:
            return []
        t0 = time.perf_counter()
        sb = self.sched.fill(self.host, kind)
        n_items, n_tokens = sb.n_items, sb.n_tokens
        decode = kind == PLAN_DECODE
        h = self.host
        # per-token causal length (prefill rows attend to positions <= their own)
        np.add(h.field("positions")[:n_tokens], 1, out=h.field("ctx_per_token")[:n_tokens])
        si = h.field("sample_index")
        samples_mask = si[:n_items] >= 0
        np.maximum(si[:n_items], 0, out=si[:n_items])
        try:
            if decode and self.use_graph:
                toks = self._decode_graph(n_items)
            else:
                self._upload(n_tokens, n_items)
                b = self._batch_views(n_tokens, n_items)
                toks = self._run_and_sample(b, decode, n_tokens, n_items, sb.req_ids)
            self.sampled_host[:n_items].copy_(toks[:n_items], non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            self.d2h_bytes_last = n_items * 4
            self.runner.ops.check()
        except Exception:
            self.sched.abort_step()
            self.metrics.failed_steps += 1
            raise
        sampled = self.sampled_host[:n_items].numpy()
        fin = self.sched.commit(sampled, self.cfg.eos_token_id)
        now = time.perf_counter()
        out = []
        for i in range(n_items):
            if not samples_mask[i]:
                continue
            r = self.requests[int(sb.req_ids[i])]
            tok = int(sampled[i])
            r.output_tokens.append(tok)
            if r.first_token_at is None:
                r.first_token_at = now
                self.metrics.observe_ttft(now - r.created_at)
            if fin[i]:
                r.finish_reason = FinishReason.EOS_TOKEN if fin[i] == 1 else FinishReason.MAX_TOKENS
                r.finished_at = now
                self.metrics.requests_finished += 1
            elif r.params.stop_sequences and self._hit_stop(r):
                self.sched.cancel(r.id)
                r.finish_reason = FinishReason.STOP_SEQUENCE
                r.finished_at = now
                self.metrics.requests_finished += 1
            if self.on_token is not None:
                self.on_token(r, tok)
            out.append(r)
        self.metrics.observe_step(decode, n_items, n_tokens, int(samples_mask.sum()), now - t0,
                                  self.sched.num_waiting, self.sched.num_running,
                                  self.sched.num_free_blocks, self.runner.num_blocks)
        return out

    @staticmethod
    def _hit_stop(r: Request) -> bool:
        for s in r.params.stop_sequences:
            if s and r.output_tokens[-len(s):] == list(s):
                return True
        return False

    def _run_and_sample(self, b, decode, n_tokens, n_items, req_ids) -> torch.Tensor:
        greedy = all(self.requests[int(i)].params.temperature <= 0 for i in req_ids)
        if greedy:
            return self.runner.forward(b, decode, n_tokens, n_items)
        logits = self.runner.forward(b, decode, n_tokens, n_items, want_logits=True)
        reqs = [self.requests[int(i)] for i in req_ids]
        return sample_tokens(logits, reqs)

    # ------------------------------------------------------------------ CUDA-graph decode
    def _bucket(self, n: int) -> int:
        for bsz in _BUCKETS:
            if bsz >= n and bsz <= self.cfg.max_num_seqs:
                return bsz
        return self.cfg.max_num_seqs

    def _decode_graph(self, n_items: int) -> torch.Tensor:
        greedy = all(self.requests[int(i)].params.temperature <= 0 for i in self.host.req_ids[:n_items])
        if not greedy:
            self._upload(n_items, n_items)
            b = self._batch_views(n_items, n_items)
            return self._run_and_sample(b, True, n_items, n_items, self.host.req_ids[:n_items])
        bsz = self._bucket(n_items)
        h = self.host
        if bsz > n_items:       # pad rows: no cache slot, no context
            h.field("token_ids")[n_items:bsz] = 0
            h.field("positions")[n_items:bsz] = 0
            h.field("slot_mapping")[n_items:bsz] = -1
            h.field("seq_lens")[n_items:bsz] = 0
            h.field("block_tables")[n_items * self.max_blocks: bsz * self.max_blocks] = 0
        self._upload(bsz, bsz)
        entry = self._graphs.get(bsz)
        if entry is None:
            b = self._batch_views(bsz, bsz)
            # warm-up outside capture (loads kernels, sizes caches), then capture
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self.runner.forward(b, True, bsz, bsz)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self.runner.forward(b, True, bsz, bsz)
            entry = (g, out)
            self._graphs[bsz] = entry
        g, out = entry
        g.replay()
        return out

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: List[List[int]], params: Optional[SamplingParams] = None,
                 max_steps: int = 1 << 30) -> List[List[int]]:
        ids = [self.add_request(p, params) for p in prompts]
        steps = 0
        while self.has_unfinished() and steps < max_steps:
            self.step()
            steps += 1
        return [self.requests[i].output_tokens for i in ids]

    def stats(self) -> Dict[str, object]:
        d = self.metrics.as_dict()
        d.update(self.sched.stats())
        return d

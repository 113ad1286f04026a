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
from collections import deque
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

class StepOutput:
    """What one iteration produced: ids of the requests that got a token, the tokens, and finish codes
    (0 running, 1 eos, 2 max_tokens).  Behaves like a sequence of ``Request`` objects."""
    __slots__ = ("_engine", "req_ids", "tokens", "finished", "_reqs")

    def __init__(self, engine, req_ids, tokens, finished, reqs=None):
        self._engine, self.req_ids, self.tokens, self.finished = engine, req_ids, tokens, finished
        self._reqs = reqs if reqs is not None else []

    def __len__(self):
        return len(self.req_ids)

    def __iter__(self):
        return iter(self._reqs)

    def __getitem__(self, k):
        return self._reqs[k]


_BUCKETS = [1, 2, 4, 8, 16, 32, 64, 96, 128, 160, 192, 224, 256, 320, 384, 448, 512, 768, 1024]


def classify_prefill_step(token_item: np.ndarray, positions: np.ndarray, n_items: int):
    """Which attention kernel a prefill step takes, from the item index and the position of each of its tokens (items
    occupy consecutive token ranges).  ``("dense", lens)``: every item is a whole prompt from position 0, attention
    reads K and V from the fused qkv buffer.  ``("paged", starts, lens, first_pos)``: some item continues a chunked
    prompt or starts behind a prefix-cache hit, the tensor-core kernel reads the paged cache; its 128-query tiles do
    not pay for a handful of tokens per item, so steps under 32 tokens per item on average return None (per-row
    kernel), as do steps whose tokens are not grouped by item."""
    n_tokens = len(token_item)
    starts = np.flatnonzero(np.diff(token_item, prepend=-1))
    if n_tokens == 0 or len(starts) != n_items:
        return None
    lens = np.diff(starts, append=n_tokens)
    first_pos = positions[starts]
    if not first_pos.any():
        return ("dense", lens)
    if n_tokens < 32 * n_items:
        return None
    return ("paged", starts, lens, first_pos)


class LLMEngine:
    def __init__(self, model, config: Optional[EngineConfig] = None, device=None, comm=None):
        """``model`` is a ``ronn_b200.Model`` (or anything with ``.graph``) holding a decoder architecture."""
        self.cfg = config or EngineConfig()
        graph = model.graph
        from .graph_match import decoder_from_graph
        self.arch, weights = decoder_from_graph(graph)     # in-tree metadata, or the decoder recognised in the operators
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
        self.runner = DecoderRunner(self.arch, weights, self.cfg, self.device, self.comm)
        self.max_blocks = self.runner.max_blocks_per_seq
        self.sched = Scheduler(self.cfg.block_size, self.runner.num_blocks, self.cfg.max_num_seqs,
                               self.cfg.max_batch_tokens, self.cfg.prefill_chunk, self.cfg.policy,
                               self.cfg.enable_prefix_cache, self.max_blocks)
        self._cpu_k = self._cpu_v = None
        if self.cfg.preemption != "recompute":
            # host block pool for swapped-out sequences: same block layout as the device cache, one pool per layer
            n_cpu = self.cfg.num_cpu_blocks or min(self.runner.num_blocks, 2048)
            self.sched.set_preemption(self.cfg.preemption, n_cpu, self.cfg.swap_min_tokens)
            shape = (n_cpu,) + tuple(self.runner.kcache[0].shape[1:])
            self._cpu_k = [torch.empty(shape, dtype=self.runner.kcache[0].dtype) for _ in self.runner.kcache]
            self._cpu_v = [torch.empty(shape, dtype=self.runner.kcache[0].dtype) for _ in self.runner.kcache]
        max_tokens = max(self.cfg.max_batch_tokens, self.cfg.max_num_seqs)
        self.host = HostBatchBuffers(max_tokens, self.cfg.max_num_seqs, self.max_blocks, pin=self.device.type == "cuda")
        self.dev_buf = torch.zeros(self.host.total, dtype=torch.int32, device=self.device)
        self.sampled_dev = torch.zeros(self.cfg.max_num_seqs, dtype=torch.int32, device=self.device)
        self.sampled_host = torch.zeros(self.cfg.max_num_seqs, dtype=torch.int32)
        self._status_host = torch.zeros(4, dtype=torch.int32)
        if self.device.type == "cuda":
            self.sampled_host = self.sampled_host.pin_memory()
            self._status_host = self._status_host.pin_memory()
        self.requests: Dict[int, Request] = {}
        # finished requests stay readable until ``release`` is called or ``max_finished_kept`` newer ones have finished
        self._finished_order: deque = deque()
        self.max_finished_kept = 4096
        self._next_id = 0
        self._graphs: Dict[int, tuple] = {}
        self.metrics = EngineMetrics()
        self.use_graph = bool(self.cfg.use_cuda_graph and self.device.type == "cuda")
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        # launcher calls of the sm_100a kernel library made for the steps of this engine (replayed graphs included)
        self.kernel_launches = 0
        self.kernel_launches_last = 0
        self.on_token: Optional[Callable[[Request, int], None]] = None
        self._non_greedy = 0
        self._watch_count = 0
        self._replayed_launches = 0
        self._h2d_sampling = 0
        self.host_seconds_last = (0.0, 0.0)
        self._part_streams: List[torch.cuda.Stream] = []
        self._part_comms: list = []
        # device-side sampling (kernel backend): per-row sampling records and the recent-token windows of the repeat
        # penalty are staged in pinned memory and reach the device in one copy per step, so that a non-greedy decode
        # step is a CUDA-graph replay like a greedy one.  Under tensor parallelism the vocabulary shards of the logits
        # are gathered first and every rank draws the same tokens from the same seeds.
        self.device_sampling = self.cfg.backend == "kernels" and self.device.type == "cuda"
        self._samp_recent = 256
        # base seed of requests that bring none; under tensor parallelism rank 0's, so that every rank draws the same tokens
        self._samp_seed = int(torch.randint(0, 2 ** 62, (1,)).item())
        if self.runner.tp > 1:
            import torch.distributed as dist
            grp = self.runner.comm.group
            t = torch.tensor([self._samp_seed], dtype=torch.int64, device=self.device)
            dist.broadcast(t, src=dist.get_global_rank(grp, 0) if grp is not None else 0, group=grp)
            self._samp_seed = int(t.item())
        if self.device_sampling:
            from ..ops import kernels as K
            n = self.cfg.max_num_seqs
            self._samp_bytes = n * K.SAMPLE_RECORD_BYTES
            self._samp_host = torch.zeros(self._samp_bytes + n * self._samp_recent * 4, dtype=torch.uint8).pin_memory()
            self._samp_dev = torch.zeros_like(self._samp_host, device=self.device)
            self._samp_counters = torch.zeros(n, dtype=torch.int64, device=self.device)

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
        r = Request(rid, toks, params, priority)
        r._token_source = self.sched.tokens
        self.requests[rid] = r
        if params.temperature > 0:
            self._non_greedy += 1
        if params.stop_sequences:
            self._watch_count += 1
        self.metrics.requests_added += 1
        return rid

    def cancel(self, request_id: int) -> bool:
        r = self.requests.get(request_id)
        if r is None or r.finished:
            return False
        self._finish(r, FinishReason.CANCELLED, time.perf_counter(), cancel=True)
        return True

    def _finish(self, r: Request, reason: FinishReason, now: float, cancel: bool = False, error: Optional[str] = None) -> None:
        """End of a request's life in the engine: its tokens are copied out of the scheduler, the scheduler forgets it
        (token history, block lists), the per-request counters are undone and the record joins the bounded list of
        finished requests."""
        r._freeze()
        if cancel:
            self.sched.cancel(r.id)
        self.sched.forget(r.id)
        r._token_source = None
        r.finish_reason = reason
        r.finished_at = now
        r.error = error
        if r.params.temperature > 0:
            self._non_greedy -= 1
        if r.params.stop_sequences:
            self._watch_count -= 1
        if not cancel:
            self.metrics.requests_finished += 1
        self._finished_order.append(r.id)
        while len(self._finished_order) > self.max_finished_kept:
            self.requests.pop(self._finished_order.popleft(), None)

    def release(self, request_id: int) -> None:
        """Drop the record of a finished request (its result has been read)."""
        r = self.requests.get(request_id)
        if r is not None and r.finished:
            del self.requests[request_id]

    def fail_unfinished(self, reason: str) -> List[int]:
        """Mark every waiting / running request as failed (used when steps keep failing); returns their ids."""
        now = time.perf_counter()
        ids = [rid for rid, r in self.requests.items() if not r.finished]
        for rid in ids:
            self._finish(self.requests[rid], FinishReason.ERROR, now, cancel=True, error=reason)
        return ids

    def _kernel_lib(self):
        if self.cfg.backend != "kernels":
            return None
        from .. import _native
        return _native.cuda()

    @property
    def _watch(self) -> bool:
        return self._watch_count > 0 or self.on_token is not None

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
        self.h2d_bytes_last = used * 4 + self._h2d_sampling
        self._h2d_sampling = 0

    def _run_swaps(self) -> None:
        """Block copies the scheduler decided on: preempted sequences go to the host pool (device -> host) before their
        device blocks are reused by this step, resumed ones come back (host -> device)."""
        if self._cpu_k is None:
            return
        o_src, o_dst, i_src, i_dst = self.sched.swaps()
        if len(o_src):
            src = torch.as_tensor(o_src, dtype=torch.long, device=self.device)
            dst = torch.as_tensor(o_dst, dtype=torch.long)
            for dev_c, cpu_c in ((self.runner.kcache, self._cpu_k), (self.runner.vcache, self._cpu_v)):
                for l in range(len(dev_c)):
                    cpu_c[l].index_copy_(0, dst, dev_c[l].index_select(0, src).cpu())
        if len(i_src):
            src = torch.as_tensor(i_src, dtype=torch.long)
            dst = torch.as_tensor(i_dst, dtype=torch.long, device=self.device)
            for dev_c, cpu_c in ((self.runner.kcache, self._cpu_k), (self.runner.vcache, self._cpu_v)):
                for l in range(len(dev_c)):
                    dev_c[l].index_copy_(0, dst, cpu_c[l].index_select(0, src).to(self.device))
        self.metrics.swapped_blocks += len(o_src) + len(i_src)

    # ------------------------------------------------------------------ one iteration
    def step(self) -> "StepOutput":
        """Run one scheduling iteration.  Returns the requests that produced a token in it."""
        kind = self.sched.schedule()
        self._run_swaps()                                # also when nothing is scheduled: a preemption may have swapped
        if kind == PLAN_NONE:
            return StepOutput(self, np.zeros(0, np.int64), np.zeros(0, np.int32), np.zeros(0, np.int32))
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
        if self.cfg.backend == "torch":
            longest = int(h.field("seq_lens")[:n_items].max())
            self.runner.step_ctx = min(-(-longest // 128) * 128, self.cfg.max_model_len)
        lib = self._kernel_lib()
        n_launch0 = lib.launches if lib is not None else 0
        self._replayed_launches = 0
        try:
            if decode and self.use_graph and self._non_greedy == 0:
                toks = self._decode_graph(n_items)
            elif decode and self.use_graph and self.device_sampling:
                self._stage_sampling(sb.req_ids[:n_items], self._bucket(n_items))
                toks = self._decode_graph(n_items, sample=True)
            else:
                self._upload(n_tokens, n_items)
                b = self._batch_views(n_tokens, n_items)
                if not decode:
                    b["dense_plan"] = self._dense_prefill_plan(n_tokens, n_items)
                toks = self._run_and_sample(b, decode, n_tokens, n_items, sb.req_ids)
            self.sampled_host[:n_items].copy_(toks[:n_items], non_blocking=True)
            status = self.runner.ops.status_tensor()
            if status is not None:                       # rides the same synchronisation as the sampled tokens
                self._status_host.copy_(status, non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            self.d2h_bytes_last = n_items * 4 + (16 if status is not None else 0)
            if status is not None and int(self._status_host[0]) != 0:
                self.runner.ops.check()                  # reads, clears and raises
        except Exception:
            self.sched.abort_step()
            self.metrics.failed_steps += 1
            raise
        self.kernel_launches_last = ((lib.launches - n_launch0) if lib is not None else 0) + self._replayed_launches
        self.kernel_launches += self.kernel_launches_last
        t_dev = time.perf_counter()
        sampled = self.sampled_host[:n_items].numpy().copy()
        req_ids = sb.req_ids.copy()
        fin = self.sched.commit(sampled, self.cfg.eos_token_id)
        now = time.perf_counter()
        if not decode:                                   # first tokens are born in prefill steps
            for i in np.nonzero(samples_mask)[0]:
                r = self.requests[int(req_ids[i])]
                if r.first_token_at is None:
                    r.first_token_at = now
                    self.metrics.observe_ttft(now - r.created_at)
        out_reqs = [self.requests[int(i)] for i in req_ids[samples_mask]]        # records survive pruning below
        for i in np.nonzero(fin)[0]:
            self._finish(self.requests[int(req_ids[i])], FinishReason.EOS_TOKEN if fin[i] == 1 else FinishReason.MAX_TOKENS, now)
        if self._watch:                                  # requests with stop sequences or a token callback
            for k, i in enumerate(np.nonzero(samples_mask)[0]):
                r = out_reqs[k]
                if r.finished:
                    if self.on_token is not None:
                        self.on_token(r, int(sampled[i]))
                    continue
                if r.params.stop_sequences and self._hit_stop(r):
                    self._finish(r, FinishReason.STOP_SEQUENCE, now, cancel=True)
                    self.metrics.requests_finished += 1
                if self.on_token is not None:
                    self.on_token(r, int(sampled[i]))
        self.metrics.observe_step(decode, n_items, n_tokens, int(samples_mask.sum()), now - t0,
                                  self.sched.num_waiting, self.sched.num_running,
                                  self.sched.num_free_blocks, self.runner.num_blocks)
        self.host_seconds_last = (t_dev - t0, now - t_dev)
        return StepOutput(self, req_ids[samples_mask], sampled[samples_mask], fin[samples_mask], out_reqs)

    @staticmethod
    def _hit_stop(r: Request) -> bool:
        for s in r.params.stop_sequences:
            if s and r.output_tokens[-len(s):] == list(s):
                return True
        return False

    def _dense_prefill_plan(self, n_tokens: int, n_items: int):
        """Index tensors for tensor-core prefill attention: over the fused qkv buffer when every item of the step is
        a whole prompt starting at position 0, over the paged cache (``"paged"`` in the plan) when items continue a
        chunked prompt or start behind a prefix-cache hit; None where the per-row paged kernel is the better fit."""
        if self.cfg.backend != "kernels" or self.device.type != "cuda" or not self.cfg.dense_prefill:
            return None
        h = self.host
        kind = classify_prefill_step(h.field("token_item")[:n_tokens], h.field("positions")[:n_tokens], n_items)
        if kind is None:
            return None
        from ..ops import kernels as K
        if kind[0] == "dense":
            return K.dense_attention_plan(kind[1].tolist(), self.device)
        _, starts, lens, first_pos = kind
        mk = lambda v: torch.tensor(np.asarray(v, dtype=np.int32), device=self.device)
        return {"paged": True, "seq_start": mk(starts), "q_len": mk(lens), "kv_len": mk(first_pos + lens),
                "max_q_len": int(lens.max()), "n_seq": n_items}

    def _run_and_sample(self, b, decode, n_tokens, n_items, req_ids) -> torch.Tensor:
        greedy = self._non_greedy == 0 or all(self.requests[int(i)].params.temperature <= 0 for i in req_ids)
        if greedy:
            return self.runner.forward(b, decode, n_tokens, n_items)
        logits = self.runner.forward(b, decode, n_tokens, n_items, want_logits=True)
        if self.device_sampling:
            self._stage_sampling(req_ids[:n_items], n_items)
            return self._sample_on_device(logits, n_items)
        reqs = [self.requests[int(i)] for i in req_ids]
        return sample_tokens(logits, reqs, base_seed=self._samp_seed if self.runner.tp > 1 else None)

    # ------------------------------------------------------------------ device-side sampling
    def _stage_sampling(self, req_ids, rows: int) -> None:
        """Fills the pinned sampling records (and the recent-token windows of rows with a repeat penalty) for the rows
        of this step and copies them to the device.  The seed of a row's draw is a function of the request's seed and
        of how many tokens it has generated, so a request samples the same tokens whatever batch it shares."""
        from ..ops import kernels as K
        buf = self._samp_host.numpy()
        rec = buf[self._samp_bytes:].view(np.int32).reshape(-1, self._samp_recent)
        any_recent = False
        for row in range(rows):
            if row < len(req_ids):
                r = self.requests[int(req_ids[row])]
                p = r.params
                n_out = self.sched.num_tokens(r.id) - len(r.prompt_tokens)
                base = p.seed if p.seed is not None else (self._samp_seed ^ (r.id * 0x9E3779B1))
                n_recent = 0
                if p.repeat_penalty != 1.0:
                    window = (r.prompt_tokens[-64:] + r.output_tokens)[-self._samp_recent:]
                    n_recent = len(window)
                    rec[row, :n_recent] = window
                    any_recent = True
                K.pack_sample_params(buf, row, p.temperature, p.top_k, p.top_p, p.repeat_penalty,
                                     (int(base) * 0x100000001B3 + n_out) & 0xFFFFFFFFFFFFFFFF, n_recent, use_counter=False)
            else:
                K.pack_sample_params(buf, row, 0.0, 0, 1.0, 1.0, 0, 0, use_counter=False)     # padded row
        used = self._samp_bytes + (rows * self._samp_recent * 4 if any_recent else 0)
        self._samp_dev[:used].copy_(self._samp_host[:used], non_blocking=True)
        self._h2d_sampling = used

    def _sample_on_device(self, logits: torch.Tensor, rows: int) -> torch.Tensor:
        from ..ops import kernels as K
        recent = self._samp_dev[self._samp_bytes:].view(torch.int32).view(-1, self._samp_recent)
        return K.sample(logits[:rows], self._samp_dev, recent, self._samp_counters)

    # ------------------------------------------------------------------ CUDA-graph decode
    def _bucket(self, n: int) -> int:
        for bsz in _BUCKETS:
            if bsz >= n and bsz <= self.cfg.max_num_seqs:
                return bsz
        return self.cfg.max_num_seqs

    def _decode_graph(self, n_items: int, sample: bool = False) -> torch.Tensor:
        bsz = self._bucket(n_items)
        h = self.host
        if bsz > n_items:       # pad rows: no cache slot, no context
            h.field("token_ids")[n_items:bsz] = 0
            h.field("positions")[n_items:bsz] = 0
            h.field("slot_mapping")[n_items:bsz] = -1
            h.field("seq_lens")[n_items:bsz] = 0
            h.field("block_tables")[n_items * self.max_blocks: bsz * self.max_blocks] = 0
        self._upload(bsz, bsz)
        key = (bsz, self.runner.step_ctx, sample)
        entry = self._graphs.get(key)
        if entry is None:
            parts = None if sample else self._split_rows(bsz)
            if sample:
                b = self._batch_views(bsz, bsz)
                run = lambda: self._sample_on_device(self.runner.forward(b, True, bsz, bsz, want_logits=True), bsz)
            elif parts is None:
                b = self._batch_views(bsz, bsz)
                run = lambda: self.runner.forward(b, True, bsz, bsz)
            else:
                views = self._batch_views(bsz, bsz)
                subs = [({k: v[r0:r1] for k, v in views.items()}, r1 - r0) for (r0, r1) in parts]
                run = lambda: self._forward_parts(subs)
            # warm-up outside capture (loads kernels, sizes caches), then capture
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                run()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            lib = self._kernel_lib()
            n0 = lib.launches if lib is not None else 0
            with torch.cuda.graph(g):
                out = run()
            entry = (g, out, (lib.launches - n0) if lib is not None else 0)
            self._graphs[key] = entry
        g, out, captured = entry
        g.replay()
        self._replayed_launches += captured
        return out

    # ------------------------------------------------------------------ concurrent part-batches of a decode step
    def _split_rows(self, bsz: int):
        """Row ranges of the part-batches of a decode step, or None when the step runs as one batch.  A decode step
        alternates HBM-bound attention with GEMMs that are too small to fill the GPU; run as independent halves on
        separate streams, the attention of one half overlaps the GEMM chain of the other."""
        n = min(int(self.cfg.decode_streams), 8)
        r = self.runner
        if n <= 1 or self.cfg.backend != "kernels" or bsz < self.cfg.decode_split_min * 2:
            return None
        if r.tp > 1 and not getattr(self.comm, "fused", False):
            return None          # library collectives of one communicator must not be issued from concurrent streams
        n = min(n, bsz // self.cfg.decode_split_min)
        # fused-collective kernels spin on their peers, so every one of them that can be in flight at once has to
        # fit on the GPU together: a part-batch stays within two row tiles (at most 64 CTAs per kernel)
        if r.tp > 1 and -(-bsz // n) > 256:
            return None
        per = -(-bsz // n)
        per = -(-per // 16) * 16
        parts = [(r0, min(r0 + per, bsz)) for r0 in range(0, bsz, per)]
        if len(parts) < 2:
            return None
        while len(self._part_streams) < len(parts):
            self._part_streams.append(torch.cuda.Stream(self.device))
        if r.tp > 1:
            while len(self._part_comms) < len(parts):        # collective: every rank reaches this at the same step
                self._part_comms.append(self.comm.clone(max_rows=1024) if self._part_comms else self.comm)
        return parts

    def _forward_parts(self, subs) -> torch.Tensor:
        """Part-batches on their own streams, each started half a layer after the previous one: part i + 1 waits for
        the first attention of part i.  Started together, the parts would run their attention kernels at the same
        time (sharing the HBM bandwidth) and then their GEMM chains at the same time (each as slow as the whole
        batch's), which gains nothing; half a layer apart, the attention of one runs under the GEMM chain of the other
        and the offset persists because both chains have the same period."""
        main = torch.cuda.current_stream()
        tp = self.runner.tp > 1
        res = []
        prev = None
        for i, (b, n) in enumerate(subs):
            st = self._part_streams[i]
            st.wait_stream(main)
            with torch.cuda.stream(st):
                if prev is not None:
                    st.wait_event(prev)
                evt = torch.cuda.Event()
                res.append(self.runner.forward(b, True, n, n, comm=self._part_comms[i] if tp else None,
                                               local_argmax=tp, on_first_attention=lambda e=evt, s=st: e.record(s)))
                prev = evt
        for i in range(len(subs)):
            main.wait_stream(self._part_streams[i])
        if tp:
            idx = torch.cat([r[0] for r in res])
            mx = torch.cat([r[1] for r in res])
            return self.runner.combine_argmax(idx, mx)
        return torch.cat(res)

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: List[List[int]], params: Optional[SamplingParams] = None,
                 max_steps: int = 1 << 30) -> List[List[int]]:
        ids = [self.add_request(p, params) for p in prompts]
        steps = 0
        while self.has_unfinished() and steps < max_steps:
            self.step()
            steps += 1
        return [self.requests[i].output_tokens for i in ids]

    @property
    def block_manager(self):
        """Page table, block metadata and pool sizes of the KV cache (``serving/cache.py``)."""
        from .cache import BlockManager
        return BlockManager(self)

    def stats(self) -> Dict[str, object]:
        d = self.metrics.as_dict()
        d.update(self.sched.stats())
        d.update(self.sched.swap_stats())
        return d

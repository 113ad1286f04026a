"""Request-level dynamic batching (crates/ronn-api/src/batch.rs:17-414).

``BatchStrategy.Static{batch_size}`` waits for exactly N requests; ``Dynamic{max_batch_size=32,
timeout_ms=10}`` takes the first request and then whatever arrives before the deadline.  Inputs are
stacked on a new leading dimension per input name, run once, and the outputs are split back per
request; an error fans out to every request of the batch.  ``BatchStats`` is actually filled.
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

import torch

from .errors import InferenceError, SessionError


@dataclass(frozen=True)
class BatchStrategy:
    kind: str = "dynamic"             # "static" | "dynamic"
    batch_size: int = 32              # static size / dynamic maximum
    timeout_ms: float = 10.0

    @staticmethod
    def static(batch_size: int) -> "BatchStrategy":
        return BatchStrategy("static", batch_size, 0.0)

    @staticmethod
    def dynamic(max_batch_size: int = 32, timeout_ms: float = 10.0) -> "BatchStrategy":
        return BatchStrategy("dynamic", max_batch_size, timeout_ms)


@dataclass
class BatchConfig:
    strategy: BatchStrategy = field(default_factory=BatchStrategy)
    queue_capacity: int = 1024
    num_workers: int = 1

    def __init__(self, strategy: Optional[BatchStrategy] = None, queue_capacity: int = 1024, num_workers: int = 1,
                 max_batch_size: Optional[int] = None, timeout_ms: Optional[float] = None):
        if strategy is None:
            strategy = BatchStrategy.dynamic(max_batch_size or 32, 10.0 if timeout_ms is None else timeout_ms)
        self.strategy = strategy
        self.queue_capacity = queue_capacity
        self.num_workers = num_workers


@dataclass
class BatchStats:
    total_requests: int = 0
    total_batches: int = 0
    total_time_ms: float = 0.0
    max_batch_seen: int = 0

    @property
    def avg_batch_size(self) -> float:
        return self.total_requests / self.total_batches if self.total_batches else 0.0

    def throughput(self) -> float:
        return self.total_requests * 1000.0 / self.total_time_ms if self.total_time_ms > 0 else 0.0

    def utilization(self, max_batch: int) -> float:
        return self.avg_batch_size / max_batch if max_batch else 0.0


class BatchProcessor:
    def __init__(self, session, config: Optional[BatchConfig] = None):
        self.session = session
        self.config = config or BatchConfig()
        self._q: "queue.Queue" = queue.Queue(maxsize=self.config.queue_capacity)
        self._stats = BatchStats()
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self._workers = [threading.Thread(target=self._worker_loop, daemon=True, name=f"ronn-batch-{i}")
                         for i in range(max(self.config.num_workers, 1))]
        for w in self._workers:
            w.start()

    # ------------------------------------------------------------------ client side
    def submit(self, inputs: Mapping[str, torch.Tensor]) -> Future:
        if self._stop.is_set():
            raise SessionError("batch processor is shut down")
        fut: Future = Future()
        try:
            self._q.put_nowait((dict(inputs), fut))
        except queue.Full:
            raise SessionError("batch queue is full") from None
        return fut

    def process_sync(self, inputs: Mapping[str, torch.Tensor], timeout: Optional[float] = None):
        return self.submit(inputs).result(timeout)

    async def process(self, inputs: Mapping[str, torch.Tensor]):
        return await asyncio.wrap_future(self.submit(inputs))

    def stats(self) -> BatchStats:
        with self._lock:
            return BatchStats(**vars(self._stats))

    def shutdown(self) -> None:
        self._stop.set()
        for w in self._workers:
            w.join(timeout=2)

    # ------------------------------------------------------------------ worker side
    def _collect(self) -> List:
        st = self.config.strategy
        try:
            first = self._q.get(timeout=0.05)
        except queue.Empty:
            return []
        batch = [first]
        if st.kind == "static":
            while len(batch) < st.batch_size and not self._stop.is_set():
                try:
                    batch.append(self._q.get(timeout=0.05))
                except queue.Empty:
                    continue
            return batch
        deadline = time.perf_counter() + st.timeout_ms / 1e3
        while len(batch) < st.batch_size:
            remaining = deadline - time.perf_counter()
            if remaining <= 0:
                break
            try:
                batch.append(self._q.get(timeout=remaining))
            except queue.Empty:
                break
        return batch

    def _worker_loop(self) -> None:
        while not self._stop.is_set():
            batch = self._collect()
            if batch:
                self._process_batch(batch)

    def _process_batch(self, batch: List) -> None:
        t0 = time.perf_counter()
        try:
            names = list(batch[0][0].keys())
            stacked = {}
            for n in names:
                ts = [torch.as_tensor(req[n]) for req, _ in batch]
                if any(t.shape != ts[0].shape for t in ts):
                    raise InferenceError(f"inputs '{n}' of the batched requests differ in shape")
                stacked[n] = torch.stack(ts, dim=0)
            # the graph sees [B, *request_shape]; a request shape with its own batch dim of 1 is folded in
            squeeze = all(v.dim() >= 2 and v.shape[1] == 1 for v in stacked.values())
            if squeeze:
                stacked = {k: v.squeeze(1) for k, v in stacked.items()}
            outs = self.session.run(stacked)
            for i, (_, fut) in enumerate(batch):
                res = {}
                for k, v in outs.items():
                    piece = v[i]
                    res[k] = piece.unsqueeze(0) if squeeze else piece
                fut.set_result(res)
        except Exception as e:
            for _, fut in batch:
                if not fut.done():
                    fut.set_exception(e if isinstance(e, InferenceError) else InferenceError(str(e)))
        ms = (time.perf_counter() - t0) * 1e3
        with self._lock:
            s = self._stats
            s.total_requests += len(batch)
            s.total_batches += 1
            s.total_time_ms += ms
            s.max_batch_seen = max(s.max_batch_seen, len(batch))

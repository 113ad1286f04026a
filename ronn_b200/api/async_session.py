"""Async facade (crates/ronn-api/src/async_session.rs:33-228): load and run on worker threads,
``run_concurrent`` over many inputs, cheap handle clones; ``AsyncBatchProcessor`` really batches
(the reference's ``infer`` is a passthrough)."""
from __future__ import annotations

import asyncio
from typing import Dict, List, Mapping, Optional

import torch

from .batch import BatchConfig, BatchProcessor, BatchStrategy
from .model import Model
from .session import InferenceSession, SessionOptions


class AsyncSession:
    def __init__(self, session: InferenceSession):
        self._session = session

    @staticmethod
    async def from_file(path) -> "AsyncSession":
        return await AsyncSession.with_options(path, SessionOptions())

    @staticmethod
    async def with_options(path, options: SessionOptions) -> "AsyncSession":
        loop = asyncio.get_running_loop()
        sess = await loop.run_in_executor(None, lambda: Model.load(path).create_session(options))
        return AsyncSession(sess)

    async def run(self, inputs: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return await self._session.run_async(inputs)

    async def run_concurrent(self, many: List[Mapping[str, torch.Tensor]]) -> List[Dict[str, torch.Tensor]]:
        return list(await asyncio.gather(*(self.run(i) for i in many)))

    def clone_handle(self) -> "AsyncSession":
        return AsyncSession(self._session)

    @property
    def session(self) -> InferenceSession:
        return self._session


class AsyncBatchProcessor:
    def __init__(self, session: AsyncSession, max_batch_size: int = 32, timeout_ms: float = 10.0):
        self._proc = BatchProcessor(session.session, BatchConfig(BatchStrategy.dynamic(max_batch_size, timeout_ms)))

    async def infer(self, inputs: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return await self._proc.process(inputs)

    def shutdown(self) -> None:
        self._proc.shutdown()

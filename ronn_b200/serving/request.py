"""Request model of the serving engine
(docs/new/RONN-Continuous-Batching-Branch-Prompt.md:84-152)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import List, Optional


class RequestState(enum.IntEnum):
    WAITING = 0
    PREFILL = 1
    DECODING = 2
    FINISHED = 3
    PREEMPTED = 4
    CANCELLED = 5


class Priority(enum.IntEnum):
    CRITICAL = 0
    HIGH = 1
    NORMAL = 2
    LOW = 3


class FinishReason(enum.Enum):
    EOS_TOKEN = "eos_token"
    MAX_TOKENS = "max_tokens"
    STOP_SEQUENCE = "stop_sequence"
    CANCELLED = "cancelled"
    ERROR = "error"


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0           # 0 = greedy
    top_k: int = 0
    top_p: float = 1.0
    repeat_penalty: float = 1.0
    stop_sequences: List[List[int]] = field(default_factory=list)
    seed: Optional[int] = None


@dataclass
class Request:
    id: int
    prompt_tokens: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    priority: Priority = Priority.NORMAL
    finish_reason: Optional[FinishReason] = None
    created_at: float = field(default_factory=time.perf_counter)
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None
    error: Optional[str] = None
    _final_tokens: Optional[List[int]] = None
    _token_source: Optional[object] = None       # callable returning prompt + generated tokens while the request is live

    @property
    def output_tokens(self) -> List[int]:
        """Generated tokens so far.  While the request is live they are read from the scheduler's token history
        (the engine does not copy tokens into Python objects on every step)."""
        if self._final_tokens is not None:
            return self._final_tokens
        if self._token_source is None:
            return []
        return self._token_source(self.id)[len(self.prompt_tokens):]

    def _freeze(self) -> None:
        if self._final_tokens is None:
            self._final_tokens = self.output_tokens

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_at is None else self.first_token_at - self.created_at

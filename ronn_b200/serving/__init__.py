"""Continuous-batching serving engine over a paged KV cache."""
from .config import EngineConfig
from .request import FinishReason, Priority, Request, RequestState, SamplingParams
from .engine import LLMEngine
from .cache import BlockLocation, BlockManager, BlockMetadata, CachePrecision, PageTable

"""``import ronn``: the module shape of the reference's Python bindings on top of ``ronn_b200``.

The reference ships a PyO3 module ``ronn`` with ``Model``, ``Session``, ``Tensor``, ``OptimizationLevel``,
``ProviderType``, ``BatchConfig`` and ``__version__`` (crates/ronn-python/src/lib.rs:47-192, model.rs:36-158,
session.rs:52-96, tensor.rs:7-40).  Code written against it keeps working: models load from a path, sessions are made
with string or enum options, ``run`` takes a dict of numpy arrays and returns a dict of numpy arrays.  Two things are
wider than the reference's code and follow its documented surface instead: arrays keep their shape (the reference
flattens everything to one dimension), and ``create_batch_processor`` / ``run_async`` / ``stats`` exist on the session.
Everything else of the runtime (providers, serving engine, tensor parallelism) is under ``ronn_b200``.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import numpy as np
import torch

import ronn_b200 as _r
from ronn_b200.api.batch import BatchConfig as _BatchConfig

__version__ = _r.__version__


class OptimizationLevel:
    """``OptimizationLevel.none() / basic() / default() / aggressive()`` (lib.rs:63-109): O0 .. O3."""
    O0, O1, O2, O3 = (_r.OptimizationLevel(i) for i in range(4))

    @staticmethod
    def none():
        return _r.OptimizationLevel.O0

    @staticmethod
    def basic():
        return _r.OptimizationLevel.O1

    @staticmethod
    def default():
        return _r.OptimizationLevel.O2

    @staticmethod
    def aggressive():
        return _r.OptimizationLevel.O3


class ProviderType:
    """``ProviderType.cpu() / gpu() / bitnet() / wasm()`` (lib.rs:111-156)."""
    CPU, GPU, BITNET, WASM = _r.ProviderType.CPU, _r.ProviderType.GPU, _r.ProviderType.BITNET, _r.ProviderType.WASM

    @staticmethod
    def cpu():
        return _r.ProviderType.CPU

    @staticmethod
    def gpu():
        return _r.ProviderType.GPU

    @staticmethod
    def bitnet():
        return _r.ProviderType.BITNET

    @staticmethod
    def wasm():
        return _r.ProviderType.WASM

    @staticmethod
    def default():
        return _r.ProviderType.CPU


def BatchConfig(max_batch_size: int = 32, timeout_ms: float = 10, queue_capacity: int = 1024):
    """Dynamic batching of up to ``max_batch_size`` requests that arrive within ``timeout_ms`` (lib.rs:159-192)."""
    return _BatchConfig(max_batch_size=max_batch_size, timeout_ms=timeout_ms, queue_capacity=queue_capacity)


class Tensor:
    """A read-only view of a tensor: ``shape()``, ``dtype()``, ``numel()`` (tensor.rs:18-40), plus ``numpy()``."""

    def __init__(self, value):
        self._t = value if isinstance(value, torch.Tensor) else torch.as_tensor(np.asarray(value))

    def shape(self):
        return list(self._t.shape)

    def dtype(self) -> str:
        return str(_r.DataType.from_torch(self._t.dtype).name).lower()

    def numel(self) -> int:
        return self._t.numel()

    def numpy(self) -> np.ndarray:
        t = self._t.detach().cpu()
        return (t.float() if t.dtype in (torch.bfloat16, torch.float16) else t).numpy()

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape()}, dtype={self.dtype()})"


class Session:
    """What ``Model.create_session`` returns: ``run({name: array}) -> {name: array}`` (session.rs:52-96)."""

    def __init__(self, inner):
        self._inner = inner

    def run(self, inputs: Mapping[str, object]) -> Dict[str, np.ndarray]:
        feeds = {k: (v._t if isinstance(v, Tensor) else torch.as_tensor(np.asarray(v))) for k, v in inputs.items()}
        return {k: Tensor(v).numpy() for k, v in self._inner.run(feeds).items()}

    async def run_async(self, inputs: Mapping[str, object]) -> Dict[str, np.ndarray]:
        feeds = {k: (v._t if isinstance(v, Tensor) else torch.as_tensor(np.asarray(v))) for k, v in inputs.items()}
        return {k: Tensor(v).numpy() for k, v in (await self._inner.run_async(feeds)).items()}

    def create_batch_processor(self, config=None):
        return self._inner.create_batch_processor(config)

    def stats(self) -> Dict[str, float]:
        return self._inner.stats()

    def input_names(self):
        return list(self._inner.input_names())

    def output_names(self):
        return list(self._inner.output_names())

    def __repr__(self) -> str:
        return f"Session(inputs={self.input_names()}, outputs={self.output_names()})"


class Model:
    """``Model.load(path)`` -> ``create_session(optimization_level="basic", provider="cpu", num_threads=None)``
    (model.rs:36-158); levels ``"O0" | "none" ... "O3" | "aggressive"``, providers ``"cpu" | "gpu" | "cuda" | "bitnet" |
    "wasm"``, or the enum values above."""

    def __init__(self, inner):
        self._inner = inner

    @staticmethod
    def load(path: str) -> "Model":
        return Model(_r.Model.load(path))

    @staticmethod
    def from_bytes(data: bytes) -> "Model":
        return Model(_r.Model.from_bytes(data))

    def input_names(self):
        return list(self._inner.input_names())

    def output_names(self):
        return list(self._inner.output_names())

    def metadata(self) -> Dict[str, object]:
        return dict(self._inner.metadata())

    def create_session(self, optimization_level="basic", provider="cpu", num_threads: Optional[int] = None,
                       enable_hrm: Optional[bool] = None) -> Session:
        return Session(self._inner.create_session(optimization_level=optimization_level, provider=provider,
                                                  num_threads=num_threads, enable_hrm=enable_hrm))

    def __repr__(self) -> str:
        return f"Model(inputs={self.input_names()}, outputs={self.output_names()})"


__all__ = ["Model", "Session", "Tensor", "OptimizationLevel", "ProviderType", "BatchConfig", "__version__"]

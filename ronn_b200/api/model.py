"""``Model``: a loaded ONNX model from which sessions are created
(crates/ronn-api/src/model.rs:9-110; documented Python surface
crates/ronn-python/README.md:19-150)."""
from __future__ import annotations

import os
from typing import Dict, List

from ..graph.ir import ModelGraph, TensorInfo
from ..onnx.loader import LoadedModel, ModelLoader
from .errors import IoError, ModelLoadError, OnnxError
from .session import InferenceSession, SessionBuilder, SessionOptions


class Model:
    def __init__(self, loaded: LoadedModel):
        self._loaded = loaded

    # ------------------------------------------------------------------ construction
    @staticmethod
    def load(path) -> "Model":
        p = os.fspath(path) if path is not None else ""
        if not p:
            raise ModelLoadError("empty model path")
        if os.path.isdir(p):
            raise ModelLoadError(f"'{p}' is a directory")
        try:
            return Model(ModelLoader.load_from_file(p))
        except IoError as e:
            raise ModelLoadError(e.message) from e
        except OnnxError as e:
            raise ModelLoadError(str(e)) from e

    @staticmethod
    def from_bytes(data: bytes) -> "Model":
        try:
            return Model(ModelLoader.load_from_bytes(data))
        except OnnxError as e:
            raise ModelLoadError(str(e)) from e

    @staticmethod
    def from_graph(graph: ModelGraph, producer_name: str = "ronn_b200") -> "Model":
        graph.validate()
        return Model(LoadedModel(graph=graph, initializers=graph.initializers, inputs=graph.inputs,
                                 outputs=graph.outputs, producer_name=producer_name, ir_version=8,
                                 opset_imports={"": 17}, metadata=dict(graph.metadata)))

    # ------------------------------------------------------------------ sessions
    def create_session_default(self) -> InferenceSession:
        return SessionBuilder(self).build()

    def create_session(self, options: SessionOptions = None, *, optimization_level=None, provider=None,
                       num_threads=None, enable_hrm=None, **kw) -> InferenceSession:
        opts = options or SessionOptions()
        if optimization_level is not None:
            opts = opts.with_optimization_level(optimization_level)
        if provider is not None:
            opts = opts.with_provider(provider)
        if num_threads is not None:
            opts = opts.with_num_threads(num_threads)
        if enable_hrm is not None:
            opts = opts.with_hrm(enable_hrm)
        for k, v in kw.items():
            if not hasattr(opts, k):
                raise TypeError(f"create_session() got an unexpected option '{k}'")
            from dataclasses import replace
            opts = replace(opts, **{k: v})
        return SessionBuilder(self).with_options(opts).build()

    # ------------------------------------------------------------------ metadata
    @property
    def graph(self) -> ModelGraph:
        return self._loaded.graph

    def producer_name(self):
        return self._loaded.producer_name

    def ir_version(self) -> int:
        return self._loaded.ir_version

    def input_names(self) -> List[str]:
        return [i.name for i in self._loaded.inputs]

    def output_names(self) -> List[str]:
        return [o.name for o in self._loaded.outputs]

    def inputs(self) -> List[TensorInfo]:
        return list(self._loaded.inputs)

    def outputs(self) -> List[TensorInfo]:
        return list(self._loaded.outputs)

    def metadata(self) -> Dict[str, object]:
        return {"producer_name": self._loaded.producer_name, "producer_version": self._loaded.producer_version,
                "ir_version": self._loaded.ir_version, "model_version": self._loaded.model_version,
                "opset_imports": dict(self._loaded.opset_imports), "node_count": len(self._loaded.graph.nodes),
                "initializer_count": len(self._loaded.initializers), **self._loaded.metadata}

    def to_bytes(self) -> bytes:
        from ..onnx.writer import model_to_bytes
        return model_to_bytes(self._loaded.graph)

    def save(self, path) -> None:
        with open(path, "wb") as f:
            f.write(self.to_bytes())

    def __repr__(self):
        return (f"Model(producer={self._loaded.producer_name!r}, ir_version={self._loaded.ir_version}, "
                f"inputs={self.input_names()}, outputs={self.output_names()})")

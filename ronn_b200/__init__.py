"""ronn_b200: a Blackwell-native ONNX inference and serving runtime.

Public surface (shape of the reference's prelude, crates/ronn-api/src/lib.rs:11-28):
``Model.load / Model.from_bytes -> create_session(SessionOptions) -> session.run({name: tensor})``.
"""
from .api.errors import (InferenceError, InvalidInput, ModelLoadError, OnnxError, ProviderError, RonnError,
                         SessionError)
from .api.model import Model
from .api.session import InferenceSession, SessionBuilder, SessionOptions
from .core.types import DataType, OptimizationLevel, ProviderType

__version__ = "0.1.0"

__all__ = ["Model", "SessionBuilder", "SessionOptions", "InferenceSession", "OptimizationLevel", "ProviderType",
           "DataType", "RonnError", "ModelLoadError", "InferenceError", "InvalidInput", "SessionError",
           "ProviderError", "OnnxError", "__version__"]

"""Error hierarchy.

Message prefixes match the reference's Display implementations
(crates/ronn-api/src/error.rs:5-33, crates/ronn-onnx/src/error.rs:6-48,
crates/ronn-core/src/error.rs:11-38).
"""
from __future__ import annotations


class RonnError(Exception):
    prefix = ""

    def __init__(self, message: str = ""):
        self.message = str(message)
        super().__init__(f"{self.prefix}{self.message}" if self.prefix else self.message)


class ModelLoadError(RonnError):
    prefix = "Failed to load model: "


class InferenceError(RonnError):
    prefix = "Inference failed: "


class InvalidInput(RonnError):
    prefix = "Invalid input: "


class SessionError(RonnError):
    prefix = "Session error: "


class ProviderError(RonnError):
    prefix = "Provider error: "


class OptimizationError(RonnError):
    prefix = "Optimization error: "


class IoError(RonnError):
    prefix = "IO error: "


class CoreError(RonnError):
    prefix = "Core error: "


class TensorError(CoreError):
    prefix = "Tensor error: "


class ShapeMismatch(CoreError):
    prefix = "Shape mismatch: "


class InvalidOperation(CoreError):
    prefix = "Invalid operation: "


class GraphError(CoreError):
    prefix = "Graph error: "


class OnnxError(RonnError):
    prefix = "ONNX error: "


class ParseError(OnnxError):
    prefix = "Failed to parse ONNX model: "


class ProtobufDecodeError(OnnxError):
    prefix = "Protobuf decode error: "


class UnsupportedIrVersion(OnnxError):
    prefix = "Unsupported IR version: "


class UnsupportedOpset(OnnxError):
    prefix = "Unsupported opset: "


class UnsupportedOperator(OnnxError):
    prefix = "Unsupported operator: "


class InvalidAttribute(OnnxError):
    prefix = "Invalid attribute: "


class ShapeInferenceError(OnnxError):
    prefix = "Shape inference error: "


class TypeConversionError(OnnxError):
    prefix = "Type conversion error: "


class MissingInput(OnnxError):
    prefix = "Missing required input: "


class InvalidGraph(OnnxError):
    prefix = "Invalid graph: "


class CommTimeoutError(RonnError):
    """A bounded device-side wait on a peer flag ran out (the kernel returned an error status)."""
    prefix = "Communication timeout: "

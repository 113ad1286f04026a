"""Synthetic-weight ONNX model builders for the benchmark configurations."""

"""ONNX model writer (serialisation through the native wire encoder).

The reference never writes models; its fixtures come from Python scripts that need the
``onnx`` package (models/create_test_models.py:11-238,
crates/ronn-api/tests/fixtures/create_fixtures.py:20-104).  That package is not a
dependency here: ``save_model`` / ``model_to_bytes`` emit the protobuf directly, which
is also how the synthetic benchmark models (ResNet-18, DistilBERT, GPT-2, BitNet) are
produced with random weights.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import numpy as np
import torch

from .. import _native
from ..graph.ir import ModelGraph, TensorInfo
from .dtypes import DataTypeMapper, tensor_to_bytes

RONN_DOMAIN = "com.ronn"


def _b(s: Optional[str]) -> bytes:
    return (s or "").encode("utf-8")


def _i64(vals):
    arr = np.asarray(list(vals), dtype=np.int64)
    return arr, arr.ctypes.data_as(_native.c_i64p)


def _strs(vals):
    arr = (C.c_char_p * max(len(vals), 1))()
    keep = [_b(v) for v in vals]
    for i, v in enumerate(keep):
        arr[i] = v
    return arr, keep


def model_to_bytes(graph: ModelGraph, ir_version: int = 8, opset: int = 17, producer_name: str = "ronn_b200",
                   producer_version: str = "0.1.0", metadata: Optional[Dict[str, str]] = None) -> bytes:
    lib = _native.host()
    h = lib.ronn_onnxw_begin(ir_version, _b(producer_name), _b(producer_version), _b(graph.name or "graph"))
    try:
        lib.ronn_onnxw_opset(h, b"", opset)
        if any(n.domain == RONN_DOMAIN for n in graph.nodes):
            lib.ronn_onnxw_opset(h, _b(RONN_DOMAIN), 1)
        md = dict(graph.metadata)
        md.update(metadata or {})
        for k, v in md.items():
            lib.ronn_onnxw_metadata(h, _b(k), _b(str(v)))
        for n in graph.nodes:
            ins, k1 = _strs(n.inputs)
            outs, k2 = _strs(n.outputs)
            lib.ronn_onnxw_node(h, _b(n.name), _b(n.op_type), _b(n.domain), ins, len(n.inputs), outs, len(n.outputs))
            for key, val in n.attributes.items():
                _write_attr(lib, h, key, val)
        for name, t in graph.initializers.items():
            _, dims = _i64(t.shape)
            raw = tensor_to_bytes(t)
            lib.ronn_onnxw_initializer(h, _b(name), DataTypeMapper.torch_to_onnx(t.dtype), dims, t.dim(), raw, len(raw))
        for kind, infos in ((0, graph.inputs), (1, graph.outputs), (2, list(graph.value_info.values()))):
            for info in infos:
                _write_value(lib, h, kind, info)
        n = C.c_uint64(0)
        p = lib.ronn_onnxw_finish(h, C.byref(n))
        return C.string_at(p, n.value)
    finally:
        lib.ronn_onnxw_free(h)


def _write_value(lib, h, kind: int, info: TensorInfo):
    keep_arr, dims = _i64(info.shape)
    params, keep = _strs([p or "" for p in info.dim_params])
    lib.ronn_onnxw_value(h, kind, _b(info.name), DataTypeMapper.to_onnx(info.data_type), len(info.shape), dims, params)


def _write_attr(lib, h, key: str, val):
    k = _b(key)
    if isinstance(val, bool):
        lib.ronn_onnxw_attr_i(h, k, int(val))
    elif isinstance(val, int):
        lib.ronn_onnxw_attr_i(h, k, val)
    elif isinstance(val, float):
        lib.ronn_onnxw_attr_f(h, k, val)
    elif isinstance(val, (str, bytes)):
        b = val if isinstance(val, bytes) else val.encode("utf-8")
        lib.ronn_onnxw_attr_s(h, k, b, len(b))
    elif isinstance(val, torch.Tensor):
        _, dims = _i64(val.shape)
        raw = tensor_to_bytes(val)
        lib.ronn_onnxw_attr_tensor(h, k, DataTypeMapper.torch_to_onnx(val.dtype), dims, val.dim(), raw, len(raw))
    elif isinstance(val, (list, tuple)):
        if len(val) and all(isinstance(v, str) for v in val):
            arr, keep = _strs(list(val))
            lib.ronn_onnxw_attr_strings(h, k, arr, len(val))
        elif any(isinstance(v, float) for v in val):
            arr = np.asarray(val, dtype=np.float32)
            lib.ronn_onnxw_attr_floats(h, k, arr.ctypes.data_as(_native.c_f32p), len(arr))
        else:
            arr, p = _i64(int(v) for v in val)
            lib.ronn_onnxw_attr_ints(h, k, p, len(arr))
    elif val is None:
        pass
    else:
        raise TypeError(f"cannot serialise attribute '{key}' of type {type(val).__name__}")


def save_model(graph: ModelGraph, path, **kw) -> None:
    data = model_to_bytes(graph, **kw)
    with open(path, "wb") as f:
        f.write(data)

"""ONNX model loader.

Behaviour follows the reference loader (crates/ronn-onnx/src/loader.rs:22-154):
IR version >= 3 required, opset < 13 only warns, initializers become tensors and are
excluded from the graph inputs, dynamic dimensions become 0, unnamed nodes are called
``node_{index}``.  Differences, all deliberate: every mapped element type is decoded
from both ``raw_data`` and the typed fields (the reference zero-fills F16/BF16 and
others, loader.rs:263-328), tensor-valued attributes are decoded instead of dropped
(loader.rs:157-195), symbolic dimension names are kept, and producer->consumer edges
exist.  The wire format is decoded by the native library.
"""
from __future__ import annotations

import ctypes as C
import json
import logging
import mmap
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .. import _native
from ..api.errors import (InvalidGraph, IoError, ParseError, ProtobufDecodeError, TypeConversionError,
                          UnsupportedIrVersion)
from ..core.types import DataType
from ..graph.ir import GraphNode, ModelGraph, TensorInfo
from .dtypes import DataTypeMapper, tensor_from_bytes

log = logging.getLogger("ronn_b200.onnx")


@dataclass
class LoadedModel:
    graph: ModelGraph
    initializers: Dict[str, torch.Tensor]
    inputs: List[TensorInfo]
    outputs: List[TensorInfo]
    producer_name: Optional[str] = None
    producer_version: Optional[str] = None
    ir_version: int = 0
    model_version: int = 0
    opset_imports: Dict[str, int] = field(default_factory=dict)
    metadata: Dict[str, str] = field(default_factory=dict)
    doc_string: str = ""
    shared_bytes: int = 0          # bytes of initializers that are views of the mapped model file (not copies)


def _fix_str(s: str) -> str:
    # the native side escapes non-ASCII bytes one by one; reassemble UTF-8 when possible
    try:
        return s.encode("latin-1").decode("utf-8")
    except (UnicodeEncodeError, UnicodeDecodeError):
        return s


def _num(v):
    if isinstance(v, str):
        return float(v)          # "nan", "inf", "-inf"
    return v


class ModelLoader:
    @staticmethod
    def load_from_file(path) -> LoadedModel:
        """The file is mapped (private, copy-on-write), parsed in place, and initializers of SHARE_BYTES or more stay
        views of the mapping: loading costs no second copy of the weights, and the ranks of a tensor-parallel job that
        load the same file share its pages and touch only the slices of the weights they move to their device."""
        path = os.fspath(path)
        try:
            with open(path, "rb") as f:
                size = os.fstat(f.fileno()).st_size
                if size == 0:
                    raise ProtobufDecodeError("empty model buffer")
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        except OSError as e:
            raise IoError(f"{e.strerror or e}: '{path}'") from None
        return ModelLoader._load(mm, memoryview(mm), os.path.dirname(os.path.abspath(path)), share=True)

    @staticmethod
    def load_from_bytes(data: bytes, base_dir: Optional[str] = None) -> LoadedModel:
        if not isinstance(data, (bytes, bytearray, memoryview)):
            raise ParseError("model data must be bytes")
        data = bytes(data)
        if len(data) == 0:
            raise ProtobufDecodeError("empty model buffer")
        return ModelLoader._load(bytearray(data), memoryview(data), base_dir, share=False)

    @staticmethod
    def _load(writable, view: memoryview, base_dir: Optional[str], share: bool) -> LoadedModel:
        """``writable``: the model bytes as an object with a writable buffer (what ctypes can point into without a
        copy); ``view``: the bytes the tensors are cut from."""
        lib = _native.host()
        n_bytes = len(view)
        buf = (C.c_uint8 * n_bytes).from_buffer(writable)
        h = lib.ronn_onnx_parse(C.cast(buf, C.c_void_p), n_bytes)
        try:
            err = lib.ronn_onnx_error(h)
            if err:
                raise ProtobufDecodeError(err.decode("utf-8", "replace"))
            n = C.c_uint64(0)
            p = lib.ronn_onnx_json(h, C.byref(n))
            doc = json.loads(C.string_at(p, n.value).decode("ascii"))
            blobs = []
            for i in range(lib.ronn_onnx_num_blobs(h)):
                bl = C.c_uint64(0)
                bp = lib.ronn_onnx_blob(h, i, C.byref(bl))
                blobs.append(C.string_at(bp, bl.value))
        finally:
            lib.ronn_onnx_free(h)
            del buf
        return _convert_model(doc, view, blobs, base_dir, share)


def _read_external(name: str, base_dir: str, loc: str, ext: Dict[str, str], dt, dims) -> bytes:
    """Bytes of an external-data tensor.  The location comes from the (untrusted) model file, so it may only name a
    regular file inside the model's own directory: absolute paths, paths that leave the directory and symbolic links
    are refused, and offset / length are checked against the file and against the tensor's declared size."""
    if os.path.isabs(loc) or loc.startswith(("/", "\\")) or (len(loc) > 1 and loc[1] == ":"):
        raise TypeConversionError(f"tensor '{name}': external data location '{loc}' is an absolute path")
    root = os.path.realpath(base_dir)
    rel = os.path.normpath(loc)
    if rel in (".", "") or rel == ".." or rel.startswith(".." + os.sep):
        raise TypeConversionError(f"tensor '{name}': external data location '{loc}' leaves the model directory")
    # every component below the model directory must be a real directory or file, never a link
    part = root
    for comp in rel.split(os.sep):
        part = os.path.join(part, comp)
        if os.path.islink(part):
            raise TypeConversionError(f"tensor '{name}': external data location '{loc}' goes through a symbolic link")
    full = os.path.realpath(part)
    if os.path.commonpath([root, full]) != root or full == root:
        raise TypeConversionError(f"tensor '{name}': external data location '{loc}' leaves the model directory")
    try:
        offset = int(ext.get("offset", 0))
        length = int(ext["length"]) if "length" in ext else None
    except ValueError as e:
        raise TypeConversionError(f"tensor '{name}': external data offset / length is not a number") from e
    count = int(np.prod(dims)) if dims else 1
    need = count * dt.itemsize
    try:
        if not os.path.isfile(full):
            raise IoError(f"tensor '{name}': external data file '{loc}' not found")
        size = os.path.getsize(full)
        if offset < 0 or offset > size or (length is not None and (length < 0 or offset + length > size)):
            raise TypeConversionError(f"tensor '{name}': external data window [{offset}, +{length}) exceeds the "
                                      f"{size}-byte file '{loc}'")
        if length is not None and length > need:
            raise TypeConversionError(f"tensor '{name}': external data length {length} exceeds the {need} bytes its "
                                      f"shape {list(dims)} holds")
        with open(full, "rb") as f:
            f.seek(offset)
            want = length if length is not None else need
            return f.read(min(want, size - offset))
    except OSError as e:
        raise IoError(f"tensor '{name}': cannot read external data file '{loc}': {e}") from e


SHARE_BYTES = 1 << 16          # initializers at least this large stay views of a mapped model file


def _tensor_from_desc(td: Dict[str, Any], data: memoryview, blobs, base_dir, share: bool = False) -> torch.Tensor:
    code = td["data_type"]
    dt = DataTypeMapper.from_onnx(code)
    dims = td["dims"]
    if any(d < 0 for d in dims):
        raise TypeConversionError(f"tensor '{_fix_str(td['name'])}' has a negative dimension {dims}")
    if td.get("external"):
        ext = {_fix_str(k): _fix_str(v) for k, v in td.get("external_data", {}).items()}
        loc = ext.get("location")
        if not loc or base_dir is None:
            raise TypeConversionError(f"tensor '{_fix_str(td['name'])}' uses external data that cannot be located")
        raw = _read_external(_fix_str(td["name"]), base_dir, loc, ext, dt, dims)
        return tensor_from_bytes(raw, dt, dims)
    if td["raw_off"] >= 0:
        raw = data[td["raw_off"]: td["raw_off"] + td["raw_len"]]
        need = dt.itemsize
        for d in dims:
            need *= int(d)
        if td["raw_len"] != need:
            raise TypeConversionError(f"tensor '{_fix_str(td['name'])}': raw_data holds {td['raw_len']} bytes, shape "
                                      f"{list(dims)} of {dt.name} needs {need}")
        return tensor_from_bytes(raw, dt, dims, share=share and need >= SHARE_BYTES)
    if td["blob"] >= 0:
        return tensor_from_bytes(blobs[td["blob"]], dt, dims)
    count = 1
    for d in dims:
        count *= int(d)
    if count == 0:
        return torch.zeros(dims, dtype=dt.torch)
    raise TypeConversionError(f"tensor '{_fix_str(td['name'])}' carries no data for {count} elements")


def _convert_attr(a: Dict[str, Any], data, blobs, base_dir):
    t = a["type"]
    if t == 1:
        return float(_num(a["f"]))
    if t == 2:
        return int(a["i"])
    if t == 3:
        return _fix_str(a["s"])
    if t == 4:
        return _tensor_from_desc(a["t"], data, blobs, base_dir)
    if t == 6:
        return [float(_num(x)) for x in a["floats"]]
    if t == 7:
        return [int(x) for x in a["ints"]]
    if t == 8:
        return [_fix_str(s) for s in a["strings"]]
    if t == 9:
        return [_tensor_from_desc(x, data, blobs, base_dir) for x in a["tensors"]]
    if t == 5:
        return {"graph": a.get("g")}
    return None     # undefined / unsupported attribute kinds carry no value


def _value_info(v: Dict[str, Any]) -> TensorInfo:
    dt = DataTypeMapper.from_onnx(v["elem_type"]) if v["elem_type"] else DataType.F32
    shape, params = [], []
    for d in (v["shape"] or []):
        if isinstance(d, str):
            shape.append(0)
            params.append(_fix_str(d) or None)
        else:
            shape.append(int(d) if d > 0 else 0)
            params.append(None)
    return TensorInfo(_fix_str(v["name"]), shape, dt, params)


def _convert_model(doc, data, blobs, base_dir, share: bool = False) -> LoadedModel:
    g = doc.get("graph")
    if g is None:
        raise InvalidGraph("Model has no graph")
    ir = int(doc.get("ir_version", 0))
    if ir < 3:
        raise UnsupportedIrVersion(f"{ir} (IR version 3 or newer is required)")
    opsets = {_fix_str(o["domain"]): int(o["version"]) for o in doc.get("opset_import", [])}
    std = opsets.get("", opsets.get("ai.onnx"))
    if std is not None and std < 13:
        log.warning("model uses opset %d; opsets below 13 are only partially supported", std)

    graph = ModelGraph()
    shared = 0
    graph.name = _fix_str(g.get("name", ""))
    for td in g["initializers"]:
        t = _tensor_from_desc(td, data, blobs, base_dir, share)
        if share and td["raw_off"] >= 0 and not td.get("external") and t.numel() * t.element_size() >= SHARE_BYTES:
            shared += t.numel() * t.element_size()
        graph.initializers[_fix_str(td["name"])] = t
    for v in g["inputs"]:
        info = _value_info(v)
        if info.name not in graph.initializers:
            graph.inputs.append(info)
    for v in g["outputs"]:
        graph.outputs.append(_value_info(v))
    for v in g.get("value_info", []):
        try:
            info = _value_info(v)
            graph.value_info[info.name] = info
        except TypeConversionError:
            pass
    for idx, nd in enumerate(g["nodes"]):
        op_type = _fix_str(nd["op_type"])
        if not op_type:
            raise InvalidGraph(f"node {idx} has no op_type")
        attrs = {}
        for a in nd["attributes"]:
            attrs[_fix_str(a["name"])] = _convert_attr(a, data, blobs, base_dir)
        name = _fix_str(nd["name"]) or f"node_{idx}"
        if std is not None and std < 13 and op_type in ("Softmax", "LogSoftmax", "Hardmax") and not nd.get("domain"):
            # before opset 13 these operators coerce their input to 2-D at `axis` (default 1)
            attrs.setdefault("axis", 1)
            attrs["legacy_flatten"] = 1
        graph.add_node(op_type, [_fix_str(s) for s in nd["inputs"]], [_fix_str(s) for s in nd["outputs"]],
                       attrs, name, _fix_str(nd.get("domain", "")))
    meta = {_fix_str(k): _fix_str(v) for k, v in doc.get("metadata_props", [])}
    graph.metadata = dict(meta)
    return LoadedModel(graph=graph, initializers=graph.initializers, inputs=graph.inputs, outputs=graph.outputs,
                       producer_name=_fix_str(doc.get("producer_name", "")) or None,
                       producer_version=_fix_str(doc.get("producer_version", "")) or None,
                       ir_version=ir, model_version=int(doc.get("model_version", 0)), opset_imports=opsets,
                       metadata=meta, doc_string=_fix_str(doc.get("doc_string", "")), shared_bytes=shared)

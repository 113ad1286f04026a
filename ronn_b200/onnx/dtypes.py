"""ONNX element-type codes <-> DataType / torch dtypes.

The ten-entry mapping is the reference's (crates/ronn-onnx/src/types.rs:6-42:
1 F32, 2 U8, 3 I8, 6 I32, 7 I64, 9 Bool, 10 F16, 11 F64, 12 U32, 16 BF16); every
other code raises TypeConversionError with the offending code in the message.
"""
from __future__ import annotations

import numpy as np
import torch

from ..api.errors import TypeConversionError
from ..core.types import DataType

_ONNX_TO_DT = {1: DataType.F32, 2: DataType.U8, 3: DataType.I8, 6: DataType.I32, 7: DataType.I64,
               9: DataType.BOOL, 10: DataType.F16, 11: DataType.F64, 12: DataType.U32, 16: DataType.BF16}
_DT_TO_ONNX = {v: k for k, v in _ONNX_TO_DT.items()}

_NAMES = {0: "UNDEFINED", 4: "UINT16", 5: "INT16", 8: "STRING", 13: "UINT64", 14: "COMPLEX64", 15: "COMPLEX128",
          17: "FLOAT8E4M3FN", 18: "FLOAT8E4M3FNUZ", 19: "FLOAT8E5M2", 20: "FLOAT8E5M2FNUZ", 21: "UINT4",
          22: "INT4", 23: "FLOAT4E2M1", 24: "FLOAT8E8M0"}


class DataTypeMapper:
    @staticmethod
    def from_onnx(code: int) -> DataType:
        try:
            return _ONNX_TO_DT[int(code)]
        except (KeyError, ValueError, TypeError):
            name = _NAMES.get(code, "unknown")
            raise TypeConversionError(f"Unsupported ONNX data type: {code} ({name})") from None

    @staticmethod
    def to_onnx(dt: DataType) -> int:
        return _DT_TO_ONNX[dt]

    @staticmethod
    def torch_to_onnx(dt: torch.dtype) -> int:
        return _DT_TO_ONNX[DataType.from_torch(dt)]


# numpy views used to reinterpret raw little-endian payloads (bf16 has no numpy dtype: go through int16)
_NP_VIEW = {DataType.F32: np.float32, DataType.U8: np.uint8, DataType.I8: np.int8, DataType.I32: np.int32,
            DataType.I64: np.int64, DataType.BOOL: np.bool_, DataType.F16: np.float16, DataType.F64: np.float64,
            DataType.U32: np.uint32, DataType.BF16: np.int16}


def tensor_from_bytes(buf, dt: DataType, shape, share: bool = False) -> torch.Tensor:
    """Build a torch tensor from little-endian bytes: its own copy, or (``share``, writable buffers only) a view of
    ``buf`` itself, which then has to outlive the tensor (a memoryview keeps its mapping alive)."""
    count = 1
    for d in shape:                 # Python integers: a declared shape may overflow 64 bits
        count *= int(d)
    need = count * dt.itemsize
    if count < 0 or len(buf) < need:
        raise TypeConversionError(f"tensor payload has {len(buf)} bytes, shape {list(shape)} of {dt.name} needs {need}")
    arr = np.frombuffer(buf, dtype=_NP_VIEW[dt], count=count)
    if not (share and count > 0 and arr.flags.writeable and arr.flags.aligned):
        arr = arr.copy()
    t = torch.from_numpy(arr)
    if dt == DataType.BF16:
        t = t.view(torch.bfloat16)
    elif dt == DataType.U32:
        t = t.view(torch.uint32) if t.dtype != torch.uint32 else t
    return t.reshape(list(shape))


def tensor_to_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().tobytes()
    return t.numpy().tobytes()

"""BitNet quantisers over the native host kernels.

Reference contracts (crates/ronn-providers/src/bitnet/quantization.rs:13-291): ``BinaryTensor`` /
``TernaryTensor`` {packed_data, shape, scale, (threshold), element_count}, ``compression_ratio``,
``get_bit`` / ``get_value``; binary = sign bit LSB-first with scale mean|x|; ternary = threshold
0.7*mean|x| with codes 00=-1, 01=0, 10=+1, four per byte.  ``method="absmean"`` adds the b1.58
weight quantiser (scale = mean|W|, q = clip(round(W/scale), -1, 1)) used by the 2-bit GPU path.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from ... import _native


class QuantizationMethod(enum.Enum):
    BINARY = "binary"
    TERNARY = "ternary"
    ASYMMETRIC = "asymmetric"     # treated as ternary with the absmean scale


def _f32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().float().cpu().numpy()
    return np.ascontiguousarray(x, dtype=np.float32)


@dataclass
class BinaryTensor:
    packed_data: np.ndarray
    shape: Tuple[int, ...]
    scale: float
    element_count: int

    def compression_ratio(self) -> float:
        return self.element_count * 4 / max(len(self.packed_data), 1)

    def get_bit(self, i: int) -> bool:
        return bool((self.packed_data[i >> 3] >> (i & 7)) & 1)

    def dequantize(self) -> torch.Tensor:
        out = np.empty(self.element_count, dtype=np.float32)
        _native.host().ronn_bitnet_dequantize_binary(self.packed_data.ctypes.data, self.element_count,
                                                     C.c_float(self.scale), out.ctypes.data)
        return torch.from_numpy(out).reshape(self.shape)


@dataclass
class TernaryTensor:
    packed_data: np.ndarray
    shape: Tuple[int, ...]
    scale: float
    threshold: float
    element_count: int

    def compression_ratio(self) -> float:
        return self.element_count * 4 / max(len(self.packed_data), 1)

    def get_value(self, i: int) -> int:
        c = (self.packed_data[i >> 2] >> (2 * (i & 3))) & 3
        return -1 if c == 0 else (1 if c == 2 else 0)

    def values(self) -> torch.Tensor:
        out = np.empty(self.element_count, dtype=np.int8)
        _native.host().ronn_bitnet_unpack_ternary(self.packed_data.ctypes.data, self.element_count, out.ctypes.data)
        return torch.from_numpy(out).reshape(self.shape)

    def dequantize(self) -> torch.Tensor:
        return self.values().float() * self.scale


def quantize_binary(x) -> BinaryTensor:
    a = _f32(x)
    n = a.size
    packed = np.zeros((n + 7) // 8, dtype=np.uint8)
    scale = _native.host().ronn_bitnet_quantize_binary(a.ctypes.data, n, packed.ctypes.data)
    return BinaryTensor(packed, tuple(a.shape), float(scale), n)


def quantize_ternary(x, method: str = "threshold") -> TernaryTensor:
    a = _f32(x)
    n = a.size
    packed = np.zeros((n + 3) // 4, dtype=np.uint8)
    if method == "absmean":
        scale = _native.host().ronn_bitnet_quantize_absmean(a.ctypes.data, n, packed.ctypes.data)
        thr = 0.5 * float(scale)
    else:
        t = C.c_float(0)
        scale = _native.host().ronn_bitnet_quantize_ternary(a.ctypes.data, n, packed.ctypes.data, C.byref(t))
        thr = t.value
    return TernaryTensor(packed, tuple(a.shape), float(scale), float(thr), n)


def pack_ternary_rows(values: torch.Tensor) -> torch.Tensor:
    """[N, K] int8 in {-1,0,1} -> [N, ceil(K/4)] uint8 (row-wise packing, the BitLinear weight format)."""
    v = np.ascontiguousarray(values.detach().cpu().numpy(), dtype=np.int8)
    n, k = v.shape
    out = np.zeros((n, (k + 3) // 4), dtype=np.uint8)
    _native.host().ronn_bitnet_pack_ternary_rows(v.ctypes.data, n, k, out.ctypes.data)
    return torch.from_numpy(out)


def unpack_ternary_rows(packed: torch.Tensor, k: int) -> torch.Tensor:
    p = np.ascontiguousarray(packed.detach().cpu().numpy(), dtype=np.uint8)
    n, stride = p.shape
    out = np.empty((n, stride * 4), dtype=np.int8)
    _native.host().ronn_bitnet_unpack_ternary(p.ctypes.data, n * stride * 4, out.ctypes.data)
    return torch.from_numpy(out[:, :k].copy())


def quantize_activations_int8(x: torch.Tensor):
    """Per-token absmax int8: returns (q int8 [rows, K], scale fp32 [rows])."""
    a = _f32(x.reshape(-1, x.shape[-1]))
    rows, cols = a.shape
    q = np.empty((rows, cols), dtype=np.int8)
    s = np.empty(rows, dtype=np.float32)
    _native.host().ronn_bitnet_quantize_act_int8(a.ctypes.data, rows, cols, q.ctypes.data, s.ctypes.data)
    return torch.from_numpy(q), torch.from_numpy(s)


def bitlinear_reference(x: torch.Tensor, w_packed: torch.Tensor, w_scale, bias: Optional[torch.Tensor], k: int,
                        n: int) -> torch.Tensor:
    """Exact-integer host evaluation of BitLinear (the oracle of the device kernel)."""
    lead = x.shape[:-1]
    q, s = quantize_activations_int8(x)
    rows = q.shape[0]
    wp = np.ascontiguousarray(w_packed.detach().cpu().numpy(), dtype=np.uint8)
    y = np.empty((rows, n), dtype=np.float32)
    ws = float(w_scale.reshape(-1)[0]) if isinstance(w_scale, torch.Tensor) else float(w_scale)
    qa, sa = q.numpy(), s.numpy()
    _native.host().ronn_bitnet_ternary_int8_matmul(qa.ctypes.data, sa.ctypes.data, wp.ctypes.data, C.c_float(ws),
                                                   y.ctypes.data, None, rows, n, k)
    out = torch.from_numpy(y)
    if bias is not None:
        out = out + bias.float().cpu()
    return out.reshape(*lead, n).to(x.dtype).to(x.device)

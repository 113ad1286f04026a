"""BitNet compute kernels: host XNOR-popcount / ternary matmuls (reference semantics,
crates/ronn-providers/src/bitnet/kernels.rs:74-319) and the BitLinear dispatch used by the decoder
(2-bit packed ternary weights x per-token int8 activations; device kernel on a GPU)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ... import _native
from .quantization import (bitlinear_reference, quantize_binary, quantize_ternary)


def binary_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """A[M,K] x B[K,N] with both operands binarised (sign, scale mean|x|), as the reference does per call."""
    M, K = a.shape
    N = b.shape[1]
    stride = (K + 7) // 8
    lib = _native.host()

    def pack_rows(m: np.ndarray) -> np.ndarray:
        bits = (m >= 0).astype(np.uint8)
        pad = stride * 8 - K
        if pad:
            bits = np.pad(bits, ((0, 0), (0, pad)))
        return np.packbits(bits, axis=1, bitorder="little")

    an = a.detach().float().cpu().numpy()
    bn = b.detach().float().cpu().numpy()
    sa, sb = float(np.abs(an).mean()), float(np.abs(bn).mean())
    ap = np.ascontiguousarray(pack_rows(an))
    bp = np.ascontiguousarray(pack_rows(bn.T.copy()))
    out = np.empty((M, N), dtype=np.float32)
    lib.ronn_bitnet_binary_matmul(ap.ctypes.data, bp.ctypes.data, out.ctypes.data, M, N, K, C.c_float(sa), C.c_float(sb))
    return torch.from_numpy(out)


def ternary_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """A[M,K] x B[K,N] with both operands ternarised by the reference's threshold quantiser."""
    M, K = a.shape
    N = b.shape[1]
    lib = _native.host()
    qa, qb = quantize_ternary(a), quantize_ternary(b.t().contiguous())
    from .quantization import pack_ternary_rows
    ap = pack_ternary_rows(qa.values().reshape(M, K)).numpy()
    bp = pack_ternary_rows(qb.values().reshape(N, K)).numpy()
    out = np.empty((M, N), dtype=np.float32)
    lib.ronn_bitnet_ternary_matmul(ap.ctypes.data, bp.ctypes.data, out.ctypes.data, M, N, K, C.c_float(qa.scale),
                                   C.c_float(qb.scale))
    return torch.from_numpy(out)


def binary_elementwise(a_packed: np.ndarray, b_packed: np.ndarray, op: str) -> np.ndarray:
    """And / Or / Xor / Nand on packed sign bits."""
    if op == "And":
        return a_packed & b_packed
    if op == "Or":
        return a_packed | b_packed
    if op == "Xor":
        return a_packed ^ b_packed
    if op == "Nand":
        return ~(a_packed & b_packed)
    raise ValueError(f"unknown packed op {op}")


def bitlinear(x: torch.Tensor, lw, backend: str = "kernels") -> torch.Tensor:
    """y = (int8(x) . ternary(W)) * x_scale * w_scale (+ bias); ``lw`` carries packed [N, K/4] uint8 + scale."""
    if x.device.type == "cuda" and backend == "kernels":
        from ...ops import bitnet as BK
        return BK.bitlinear(x, lw.packed, lw.scale, lw.bias, lw.k, lw.n)
    if x.device.type == "cuda":
        # library baseline: dequantise to the activation dtype and use a dense matmul on quantised activations
        from .quantization import unpack_ternary_rows
        if getattr(lw, "_dense", None) is None:
            lw._dense = unpack_ternary_rows(lw.packed, lw.k).to(x.device, x.dtype)
        xf = x.float()
        s = xf.abs().amax(-1, keepdim=True).clamp_min(1e-5) / 127.0
        q = torch.round(xf / s).clamp(-127, 127)
        y = torch.matmul(q.to(x.dtype), lw._dense.t()).float() * s * float(lw.scale)
        if lw.bias is not None:
            y = y + lw.bias.float()
        return y.to(x.dtype)
    return bitlinear_reference(x, lw.packed, lw.scale, lw.bias, lw.k, lw.n)

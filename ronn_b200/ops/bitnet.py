"""Launch wrappers of the BitNet device kernels (activation quantisation, ternary x int8 BitLinear, packing)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from .kernels import KernelError, _DT, _check, _ptr, _stream, status_word


def act_quant_int8(x: torch.Tensor):
    """Per-token absmax quantisation: returns (q int8 [rows, K], scale fp32 [rows])."""
    K = x.shape[-1]
    x2 = x.reshape(-1, K).contiguous()
    rows = x2.shape[0]
    q = torch.empty((rows, K), dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    status_word(x.device)
    _check(_native.cuda().ronn_act_quant_int8(x2.data_ptr(), q.data_ptr(), s.data_ptr(), rows, K, _DT[x.dtype], _stream()),
           "act_quant_int8")
    return q, s


def rmsnorm_quant_int8(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-5):
    """RMSNorm followed by per-token int8 quantisation in one pass: returns (q, scale)."""
    K = x.shape[-1]
    x2 = x.reshape(-1, K).contiguous()
    rows = x2.shape[0]
    q = torch.empty((rows, K), dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    status_word(x.device)
    _check(_native.cuda().ronn_norm_quant_int8(x2.data_ptr(), gamma.data_ptr(), q.data_ptr(), s.data_ptr(), None, rows, K,
                                               float(eps), _DT[x.dtype], _stream()), "norm_quant_int8")
    return q, s


def swiglu_quant_int8(x: torch.Tensor):
    """x = [rows, 2F] (gate | up) -> int8 quantisation of silu(gate) * up in one pass: (q [rows, F], scale [rows])."""
    F2 = x.shape[-1]
    xc = x.reshape(-1, F2).contiguous()
    rows, F = xc.shape[0], F2 // 2
    q = torch.empty((rows, F), dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(_native.cuda().ronn_swiglu_quant_int8(xc.data_ptr(), q.data_ptr(), s.data_ptr(), rows, F, _DT[x.dtype], _stream()),
           "swiglu_quant_int8")
    return q, s


_WS_BYTES = {}


def slice_workspace(M: int, n: int, k: int, device) -> Optional[torch.Tensor]:
    """Scratch memory for the K slices of a skinny BitLinear call (None when the shape is not sliced).  A fresh tensor per
    call: calls on concurrent streams must not share it, and inside a CUDA-graph capture it comes from the graph's pool."""
    key = (M, n, k)
    nbytes = _WS_BYTES.get(key)
    if nbytes is None:
        nbytes = int(_native.cuda().ronn_bitlinear_workspace_bytes(M, n, k))
        _WS_BYTES[key] = nbytes
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def bitlinear_q(q: torch.Tensor, x_scale: torch.Tensor, w_packed: torch.Tensor, w_scale: float,
                bias: Optional[torch.Tensor], n: int, k: int, out_dtype: torch.dtype) -> torch.Tensor:
    """int8 activations [M, K] x packed ternary weights [N, K/4] -> [M, N] in out_dtype."""
    M = q.shape[0]
    if w_packed.dtype != torch.uint8 or w_packed.shape != (n, k // 4) or not w_packed.is_contiguous():
        raise KernelError(f"packed weight must be contiguous uint8 [{n}, {k // 4}], got {tuple(w_packed.shape)}")
    out = torch.empty((M, n), dtype=out_dtype, device=q.device)
    if bias is not None and bias.dtype != out_dtype:
        bias = bias.to(out_dtype)
    ws = slice_workspace(M, n, k, q.device)
    _check(_native.cuda().ronn_bitlinear(q.data_ptr(), w_packed.data_ptr(), x_scale.data_ptr(), float(w_scale), _ptr(bias),
                                         out.data_ptr(), _ptr(ws), M, n, k, q.stride(0), _DT[out_dtype],
                                         status_word(q.device).data_ptr(), _stream()), "bitlinear")
    return out


def bitlinear(x: torch.Tensor, w_packed: torch.Tensor, w_scale, bias: Optional[torch.Tensor], k: int, n: int) -> torch.Tensor:
    """y = (int8(x) . ternary(W)) * x_scale * w_scale (+ bias) for x [..., K] in bf16/fp16."""
    lead = x.shape[:-1]
    q, s = act_quant_int8(x)
    ws = float(w_scale.reshape(-1)[0]) if isinstance(w_scale, torch.Tensor) else float(w_scale)
    return bitlinear_q(q, s, w_packed, ws, bias, n, k, x.dtype).reshape(*lead, n)


def ternary_pack(values: torch.Tensor) -> torch.Tensor:
    """int8 {-1,0,1} [rows, K] on the device -> packed uint8 [rows, K/4]."""
    rows, K = values.shape
    v = values.contiguous()
    out = torch.empty((rows, K // 4), dtype=torch.uint8, device=values.device)
    _check(_native.cuda().ronn_ternary_pack(v.data_ptr(), out.data_ptr(), rows, K, _stream()), "ternary_pack")
    return out

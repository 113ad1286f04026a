"""Fused skinny GEMM: split-K tcgen05 GEMM + row reduction + bias / activation / residual + LayerNorm / RMSNorm in
ONE launch (``csrc/kernels/gemm_fuse.cu``).

``gemm_fuse`` is the single-GPU form: the K slices of a decode-sized projection are summed, finished and normalised
by the kernel that computed them, so a transformer half-block (projection + bias + residual + next norm) is one
launch.  The tensor-parallel form of the same kernel lives in ``parallel/symm.py``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from .. import _native
from .kernels import KernelError, _ACT, _DT, status_word

MAX_RANKS = 8


class FuseParams(C.Structure):
    """Mirror of ``RonnGemmFuseParams`` (csrc/kernels/gemm_fuse.h)."""
    _fields_ = [
        ("A", C.c_void_p), ("W", C.c_void_p),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("lda", C.c_int), ("ldw", C.c_int),
        ("splitk", C.c_int), ("bn", C.c_int), ("dtype", C.c_int),
        ("part", C.c_void_p * MAX_RANKS), ("part_mc", C.c_void_p), ("parity_stride", C.c_long),
        ("flags", C.c_void_p * MAX_RANKS), ("flags_mc", C.c_void_p), ("state", C.c_void_p),
        ("rank", C.c_int), ("world", C.c_int), ("nvls", C.c_int), ("scatter", C.c_int),
        ("out", C.c_void_p * MAX_RANKS), ("out_mc", C.c_void_p),
        ("norm_out", C.c_void_p * MAX_RANKS), ("norm_mc", C.c_void_p), ("ld_out", C.c_long),
        ("bias", C.c_void_p), ("residual", C.c_void_p), ("ld_res", C.c_long),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("eps", C.c_float),
        ("norm_mode", C.c_int), ("act", C.c_int), ("wait_seconds", C.c_double), ("trace", C.c_void_p),
    ]


class LLParams(C.Structure):
    """Mirror of ``RonnGemmLLParams`` (csrc/kernels/gemm_ll.h)."""
    _fields_ = [
        ("A", C.c_void_p), ("W", C.c_void_p),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("lda", C.c_int), ("ldw", C.c_int),
        ("bn", C.c_int), ("splitk", C.c_int), ("dtype", C.c_int),
        ("scatter_area", C.c_void_p * MAX_RANKS), ("scatter_parity_stride", C.c_long),
        ("result_area", C.c_void_p * MAX_RANKS), ("result_mc", C.c_void_p), ("result_parity_stride", C.c_long),
        ("state", C.c_void_p), ("rank", C.c_int), ("world", C.c_int), ("nvls", C.c_int),
        ("out", C.c_void_p), ("norm_out", C.c_void_p), ("ld_out", C.c_long),
        ("bias", C.c_void_p), ("residual", C.c_void_p), ("ld_res", C.c_long),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("eps", C.c_float), ("norm_mode", C.c_int),
        ("wait_seconds", C.c_double), ("trace", C.c_void_p), ("phases", C.c_int),
        ("quant_out", C.c_void_p), ("quant_scale", C.c_void_p),
    ]


class BitLinearLLParams(C.Structure):
    """Mirror of ``RonnBitLinearLLParams`` (csrc/kernels/gemm_ll.h)."""
    _fields_ = [("xq", C.c_void_p), ("w_packed", C.c_void_p), ("x_scale", C.c_void_p), ("w_scale", C.c_float),
                ("ldx", C.c_int), ("ll", LLParams)]


_NORM = {"": 0, None: 0, "none": 0, "layernorm": 1, "rmsnorm": 2}
_LOCAL = {}


def _lib():
    lib = _native.cuda()
    if not getattr(lib, "_fuse_declared", False):
        lib.ronn_gemm_fuse.restype = C.c_int
        lib.ronn_gemm_fuse.argtypes = [C.POINTER(FuseParams), C.c_void_p, C.c_void_p]
        lib.ronn_gemm_fuse_state_ints.restype = C.c_int
        lib.ronn_gemm_fuse_flag_ints.restype = C.c_int
        lib.ronn_gemm_ll.restype = C.c_int
        lib.ronn_gemm_ll.argtypes = [C.POINTER(LLParams), C.c_void_p, C.c_void_p]
        lib.ronn_bitlinear_ll.restype = C.c_int
        lib.ronn_bitlinear_ll.argtypes = [C.POINTER(BitLinearLLParams), C.c_void_p, C.c_void_p]
        lib._fuse_declared = True
    return lib


class _LocalScratch:
    """Per (device, stream) scratch of the single-GPU form: fp32 partial sums (two parity slots), the row-tile
    counters and the state block.  Launches on one stream are ordered, so they can share it."""

    def __init__(self, dev: torch.device, floats: int):
        lib = _lib()
        self.parity_stride = floats
        self.part = torch.empty(2 * floats, dtype=torch.float32, device=dev)
        self.flags = torch.zeros(lib.ronn_gemm_fuse_flag_ints(), dtype=torch.int32, device=dev)
        self.state = torch.zeros(lib.ronn_gemm_fuse_state_ints(), dtype=torch.int32, device=dev)


def _scratch(dev: torch.device, floats: int) -> _LocalScratch:
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    s = _LOCAL.get(key)
    if s is None or s.parity_stride < floats:
        # a larger area replaces the old one; counters and state start from zero again, which is consistent because
        # both are only ever compared with each other
        s = _LocalScratch(dev, max(floats, 1 << 21))
        _LOCAL[key] = s
    return s


def pick_splitk(M: int, N: int, K: int, sms: int = 148) -> int:
    """K slices for a decode-sized projection: enough tiles for about one CTA per SM (at most two), at least two
    64-wide K blocks per slice."""
    kb = (K + 63) // 64
    m_tiles = (M + 127) // 128
    best = 1
    for s in (1, 2, 4, 8, 16):
        if s > kb or kb // s < 2:
            break
        tiles64 = m_tiles * ((N + 63) // 64) * s
        best = s
        if tiles64 >= sms:
            break
    return best


def gemm_fuse(a: torch.Tensor, w_nk: torch.Tensor, bias: Optional[torch.Tensor] = None,
              residual: Optional[torch.Tensor] = None, norm: Optional[Tuple] = None, activation: str = "",
              splitk: int = 0, bn: int = 0, out: Optional[torch.Tensor] = None,
              norm_out: Optional[torch.Tensor] = None, trace: Optional[torch.Tensor] = None):
    """x = act(a @ w_nk^T + bias) + residual and, with ``norm=(kind, gamma, beta, eps)``, h = norm(x), in one launch.
    Returns x, or (x, h).  ``splitk`` 0 picks the slice count from the shape."""
    if a.dim() != 2 or w_nk.dim() != 2 or a.shape[1] != w_nk.shape[1]:
        raise KernelError(f"gemm_fuse shape mismatch: a {tuple(a.shape)} w {tuple(w_nk.shape)}")
    if a.dtype not in (torch.bfloat16, torch.float16) or w_nk.dtype != a.dtype:
        raise KernelError("gemm_fuse needs bf16/fp16 operands of one dtype")
    if a.stride(1) != 1 or w_nk.stride(1) != 1:
        raise KernelError("gemm_fuse operands must be K-contiguous")
    M, Kd = a.shape
    N = w_nk.shape[0]
    S = splitk if splitk > 0 else pick_splitk(M, N, Kd)
    sc = _scratch(a.device, S * M * N)
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    if residual is not None and residual.stride(1) != 1:
        residual = residual.contiguous()
    if bias is not None and bias.dtype != a.dtype:
        bias = bias.to(a.dtype)
    p = FuseParams()
    p.A, p.W = a.data_ptr(), w_nk.data_ptr()
    p.M, p.N, p.K, p.lda, p.ldw = M, N, Kd, a.stride(0), w_nk.stride(0)
    p.splitk, p.bn, p.dtype = S, bn, _DT[a.dtype]
    p.part[0], p.parity_stride = sc.part.data_ptr(), sc.parity_stride
    p.flags[0], p.state = sc.flags.data_ptr(), sc.state.data_ptr()
    p.rank, p.world, p.nvls, p.scatter = 0, 1, 0, 0
    p.out[0], p.ld_out = out.data_ptr(), out.stride(0)
    p.bias = None if bias is None else bias.data_ptr()
    p.residual = None if residual is None else residual.data_ptr()
    p.ld_res = residual.stride(0) if residual is not None else 0
    p.act = _ACT[activation]
    p.wait_seconds = 2.0
    p.trace = None if trace is None else trace.data_ptr()
    if norm is not None:
        kind, gamma, beta, eps = norm
        if norm_out is None:
            norm_out = torch.empty_like(out)
        if norm_out.stride(0) != out.stride(0):
            raise KernelError("gemm_fuse: x and h must share a row stride")
        p.norm_mode, p.eps = _NORM[kind], float(eps)
        p.gamma = None if gamma is None else gamma.data_ptr()
        p.beta = None if beta is None else beta.data_ptr()
        p.norm_out[0] = norm_out.data_ptr()
    rc = _lib().ronn_gemm_fuse(C.byref(p), status_word(a.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise KernelError(f"gemm_fuse failed with code {rc} (M={M}, N={N}, K={Kd}, splitk={S}, bn={bn})")
    return out if norm is None else (out, norm_out)

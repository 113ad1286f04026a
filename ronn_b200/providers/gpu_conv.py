"""Convolution / pooling resolution of the GPU provider: NHWC nodes go to the implicit-GEMM tcgen05 kernel."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..graph.ir import GraphNode
from ..ops import kernels as K
from .. import _native

_HALF = (torch.bfloat16, torch.float16)


def _ints(v, n, default):
    if v is None:
        return [default] * n
    return [int(x) for x in v]


def conv2d_nhwc(x, w, bias=None, residual=None, stride=1, pad=0, dil=1, relu=False, out=None, out_hw=None):
    """x [N,H,W,C], w [Cout,R,S,C] (C % 8 == 0, Cout % 8 == 0) -> [N,Ho,Wo,Cout]; bias/residual/ReLU fused.
    ``pad`` is the top/left padding; ``out_hw`` overrides the output size computed for symmetric padding (taps that
    fall outside the input read zeros either way)."""
    N, H, W, C = x.shape
    Cout, R, S, Cw = w.shape
    if Cw != C or C % 8 or Cout % 8:
        raise K.KernelError(f"conv2d_nhwc needs matching channels that are multiples of 8 (x {tuple(x.shape)}, w {tuple(w.shape)})")
    if out_hw is not None:
        Ho, Wo = out_hw
    else:
        Ho = (H + 2 * pad - dil * (R - 1) - 1) // stride + 1
        Wo = (W + 2 * pad - dil * (S - 1) - 1) // stride + 1
    x = x.contiguous()
    if out is None:
        out = torch.empty((N, Ho, Wo, Cout), dtype=x.dtype, device=x.device)
    if residual is not None:
        residual = residual.contiguous()
    ws = K.splitk_workspace(x.device, 1 << 22)      # fp32 scratch for the split-K form of the deep layers
    rc = _native.cuda().ronn_conv2d(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(),
                                    None if residual is None else residual.data_ptr(), out.data_ptr(), N, H, W, C, Cout,
                                    R, S, stride, pad, dil, Ho, Wo, 1 if relu else 0, 0 if x.dtype == torch.bfloat16 else 1,
                                    ws.data_ptr(), ws.numel(),
                                    K.status_word(x.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise K.KernelError(f"conv2d failed with code {rc}")
    return out


def stem_weights_s2d(w: torch.Tensor) -> torch.Tensor:
    """[Cout, 7, 7, C] (C <= 4) weights of a stride-2, pad-3 convolution -> [Cout, 4, 4, 16] weights of the equivalent
    stride-1 convolution over the 2x2 space-to-depth input (top/left padding 2): block tap (b, bx) and sub-pixel
    (dy, dx) hold original tap (2 b + dy - 1, 2 bx + dx - 1); taps outside the 7x7 window are zero."""
    Cout, R, S, C = w.shape
    w2 = torch.zeros((Cout, 4, 4, 16), dtype=w.dtype, device=w.device)
    for b in range(4):
        for dy in range(2):
            r = 2 * b + dy - 1
            if not 0 <= r < R:
                continue
            for bx in range(4):
                for dx in range(2):
                    s_ = 2 * bx + dx - 1
                    if 0 <= s_ < S:
                        q = dy * 2 + dx
                        w2[:, b, bx, q * C:(q + 1) * C] = w[:, r, s_, :]
    return w2.contiguous()


def stem_conv_s2d(x_nchw, w2, bias, relu):
    """7x7 / stride 2 / pad 3 first convolution of an image network from the NCHW input: one kernel rearranges the input
    into its 2x2 space-to-depth NHWC form, the implicit-GEMM kernel then runs a 4x4 stride-1 convolution with K = 256."""
    N, C, H, W = x_nchw.shape
    x2 = torch.empty((N, H // 2, W // 2, 16), dtype=x_nchw.dtype, device=x_nchw.device)
    rc = _native.cuda().ronn_nchw_to_s2d16(x_nchw.data_ptr(), x2.data_ptr(), N, C, H, W,
                                           0 if x_nchw.dtype == torch.bfloat16 else 1,
                                           torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise K.KernelError(f"nchw_to_s2d16 failed with code {rc}")
    return conv2d_nhwc(x2, w2, bias, None, 1, 2, 1, relu, out_hw=(H // 2, W // 2))


def maxpool_nhwc(x, k, stride, pad):
    N, H, W, C = x.shape
    Ho, Wo = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    x = x.contiguous()
    y = torch.empty((N, Ho, Wo, C), dtype=x.dtype, device=x.device)
    rc = _native.cuda().ronn_maxpool_nhwc(x.data_ptr(), y.data_ptr(), N, H, W, C, Ho, Wo, k, stride, pad,
                                          0 if x.dtype == torch.bfloat16 else 1, torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise K.KernelError(f"maxpool failed with code {rc}")
    return y


def global_avgpool_nhwc(x):
    N, H, W, C = x.shape
    x = x.contiguous()
    y = torch.empty((N, 1, 1, C), dtype=x.dtype, device=x.device)
    rc = _native.cuda().ronn_global_avgpool_nhwc(x.data_ptr(), y.data_ptr(), N, H * W, C,
                                                 0 if x.dtype == torch.bfloat16 else 1, torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise K.KernelError(f"global_avgpool failed with code {rc}")
    return y


def conv_resolver(table, node: GraphNode, fallback):
    a = node.attributes
    strides, dil = _ints(a.get("strides"), 2, 1), _ints(a.get("dilations"), 2, 1)
    pads = _ints(a.get("pads"), 4, 0)
    simple = (strides[0] == strides[1] and dil[0] == dil[1] and len(set(pads)) == 1 and int(a.get("group", 1)) == 1
              and a.get("auto_pad", "NOTSET") == "NOTSET" and a.get("activation", "") in ("", "Relu"))
    if not simple:
        return fallback
    relu = a.get("activation", "") == "Relu"
    cache = {}

    def run(i, attrs, c):
        x, w = i[0], i[1]
        if x.dtype not in _HALF or w.dtype != x.dtype or w.shape[0] % 8:
            return fallback(i, attrs, c)
        C = x.shape[-1]
        if (C <= 4 and tuple(w.shape[1:3]) == (7, 7) and strides[0] == 2 and pads[0] == 3 and dil[0] == 1
                and len(i) <= 3 and x.shape[1] % 2 == 0 and x.shape[2] % 2 == 0
                and x.permute(0, 3, 1, 2).is_contiguous()):
            if "w2" not in cache:
                cache["w2"] = stem_weights_s2d(w)
            return [stem_conv_s2d(x.permute(0, 3, 1, 2), cache["w2"], i[2] if len(i) > 2 else None, relu)]
        if C % 8:                                   # e.g. the 3-channel stem: zero channels keep the result unchanged
            padc = 8 - C % 8
            if "w" not in cache:
                cache["w"] = F.pad(w, (0, padc)).contiguous()
            w = cache["w"]
            nchw = x.permute(0, 3, 1, 2)
            if C < 8 and nchw.is_contiguous():
                # an NHWC view of NCHW memory (the graph input after the layout pass): convert and pad in one kernel
                n_, h_, w_ = x.shape[0], x.shape[1], x.shape[2]
                xp = torch.empty((n_, h_, w_, 8), dtype=x.dtype, device=x.device)
                rc = _native.cuda().ronn_nchw_to_nhwc8(nchw.data_ptr(), xp.data_ptr(), n_, C, h_, w_,
                                                       0 if x.dtype == torch.bfloat16 else 1,
                                                       torch.cuda.current_stream().cuda_stream)
                if rc != 0:
                    raise K.KernelError(f"nchw_to_nhwc8 failed with code {rc}")
                x = xp
            else:
                x = F.pad(x, (0, padc))
        bias = i[2] if len(i) > 2 else None
        res = i[3] if len(i) > 3 else None
        return [conv2d_nhwc(x, w, bias, res, strides[0], pads[0], dil[0], relu)]
    return run


def pool_resolver(table, node: GraphNode, fallback):
    a = node.attributes
    if node.op_type == "GlobalAveragePool":
        def run_gap(i, attrs, c):
            x = i[0]
            if x.dtype not in _HALF or x.shape[-1] % 8:
                return fallback(i, attrs, c)
            return [global_avgpool_nhwc(x)]
        return run_gap
    k = _ints(a.get("kernel_shape"), 2, 2)
    s = _ints(a.get("strides"), 2, 1)
    p = _ints(a.get("pads"), 4, 0)
    if k[0] != k[1] or s[0] != s[1] or len(set(p)) != 1 or int(a.get("ceil_mode", 0)) or a.get("dilations") not in (None, [1, 1]):
        return fallback

    def run(i, attrs, c):
        x = i[0]
        if x.dtype not in _HALF or x.shape[-1] % 8:
            return fallback(i, attrs, c)
        return [maxpool_nhwc(x, k[0], s[0], p[0])]
    return run

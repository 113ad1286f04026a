"""More standard ONNX operators, registered into the same table as ``registry.py``.

The reference stops at 39 operators (crates/ronn-onnx/src/ops/mod.rs:50-139); exported vision and language models use
many more.  These follow the ONNX operator specification (opset 17 attribute / input conventions) and run on torch
tensors, so they serve the CPU provider and the GPU provider's fallback path alike.
"""
from __future__ import annotations

import math
from typing import List

import torch
import torch.nn.functional as F

from ..api.errors import InvalidAttribute, InvalidGraph
from .registry import _ints, _reduce, _unary, op

# ------------------------------------------------------------------------------ element-wise
_unary("Sin", torch.sin)
_unary("Cos", torch.cos)
_unary("Round", torch.round)                      # half to even, as ONNX specifies
_unary("IsNaN", torch.isnan)
_unary("Mish", lambda x: x * torch.tanh(F.softplus(x)))
_unary("HardSwish", lambda x: x * torch.clamp(x / 6.0 + 0.5, 0.0, 1.0))
_unary("Softsign", lambda x: x / (1 + x.abs()))


@op("IsInf", 1)
def _isinf(i, a, c):
    x = i[0]
    pos, neg = int(a.get("detect_positive", 1)), int(a.get("detect_negative", 1))
    out = torch.zeros_like(x, dtype=torch.bool)
    if pos:
        out |= torch.isposinf(x)
    if neg:
        out |= torch.isneginf(x)
    return [out]


@op("Selu", 1)
def _selu(i, a, c):
    alpha, gamma = float(a.get("alpha", 1.6732632423543772)), float(a.get("gamma", 1.0507009873554805))
    x = i[0]
    return [gamma * torch.where(x > 0, x, alpha * (torch.exp(x) - 1))]


@op("Celu", 1)
def _celu(i, a, c):
    return [F.celu(i[0], alpha=float(a.get("alpha", 1.0)))]


@op("ThresholdedRelu", 1)
def _thresholded_relu(i, a, c):
    x = i[0]
    return [torch.where(x > float(a.get("alpha", 1.0)), x, torch.zeros_like(x))]


@op("Shrink", 1)
def _shrink(i, a, c):
    x, lambd, bias = i[0], float(a.get("lambd", 0.5)), float(a.get("bias", 0.0))
    return [torch.where(x < -lambd, x + bias, torch.where(x > lambd, x - bias, torch.zeros_like(x)))]


@op("PRelu", 2)
def _prelu(i, a, c):
    x, slope = i
    return [torch.where(x >= 0, x, x * slope)]


@op("Mod", 2)
def _mod(i, a, c):
    x, y = i
    if int(a.get("fmod", 0)):
        return [torch.fmod(x, y)]                 # sign of the dividend
    return [torch.remainder(x, y)]                # sign of the divisor (integer semantics of ONNX Mod)


@op("Mean", 1, None)
def _mean(i, a, c):
    out = i[0]
    for t in i[1:]:
        out = out + t
    return [out / len(i)]


@op("Hardmax", 1)
def _hardmax(i, a, c):
    x, axis = i[0], int(a.get("axis", -1))
    idx = x.argmax(dim=axis, keepdim=True)
    return [torch.zeros_like(x).scatter_(axis, idx, 1.0)]


# ------------------------------------------------------------------------------ reductions
op("ReduceL1", 1, 2)(_reduce(lambda x, ax, k: x.abs().sum(dim=ax, keepdim=k)))
op("ReduceSumSquare", 1, 2)(_reduce(lambda x, ax, k: x.pow(2).sum(dim=ax, keepdim=k)))
op("ReduceLogSum", 1, 2)(_reduce(lambda x, ax, k: x.sum(dim=ax, keepdim=k).log()))
op("ReduceLogSumExp", 1, 2)(_reduce(lambda x, ax, k: torch.logsumexp(x, dim=ax, keepdim=k)))


@op("CumSum", 2)
def _cumsum(i, a, c):
    x, axis = i[0], int(_ints(i[1])[0])
    exclusive, reverse = int(a.get("exclusive", 0)), int(a.get("reverse", 0))
    if reverse:
        x = x.flip(axis)
    y = x.cumsum(axis)
    if exclusive:
        y = y - x
    return [y.flip(axis) if reverse else y]


@op("TopK", 2)
def _topk(i, a, c):
    x, k = i[0], int(_ints(i[1])[0])
    axis, largest, sorted_ = int(a.get("axis", -1)), bool(int(a.get("largest", 1))), bool(int(a.get("sorted", 1)))
    v, idx = torch.topk(x, k, dim=axis, largest=largest, sorted=sorted_)
    return [v, idx.to(torch.int64)]


@op("LpNormalization", 1)
def _lpnorm(i, a, c):
    x, axis, p = i[0], int(a.get("axis", -1)), int(a.get("p", 2))
    if p not in (1, 2):
        raise InvalidAttribute("LpNormalization supports p = 1 or 2")
    n = x.abs().sum(dim=axis, keepdim=True) if p == 1 else x.pow(2).sum(dim=axis, keepdim=True).sqrt()
    return [x / n]


# ------------------------------------------------------------------------------ normalisation / convolution family
@op("InstanceNormalization", 3)
def _instance_norm(i, a, c):
    x, scale, bias = i
    return [F.instance_norm(x, weight=scale, bias=bias, eps=float(a.get("epsilon", 1e-5)))]


@op("GroupNormalization", 3)
def _group_norm(i, a, c):
    x, scale, bias = i
    groups = int(a["num_groups"])
    if scale.numel() == groups and x.shape[1] != groups:       # opset 18 gives one scale per group
        rep = x.shape[1] // groups
        scale, bias = scale.repeat_interleave(rep), bias.repeat_interleave(rep)
    return [F.group_norm(x, groups, scale, bias, eps=float(a.get("epsilon", 1e-5)))]


@op("LRN", 1)
def _lrn(i, a, c):
    return [F.local_response_norm(i[0], int(a["size"]), alpha=float(a.get("alpha", 1e-4)),
                                  beta=float(a.get("beta", 0.75)), k=float(a.get("bias", 1.0)))]


@op("ConvTranspose", 2, 3)
def _conv_transpose(i, a, c):
    x, w = i[0], i[1]
    b = i[2] if len(i) > 2 else None
    nd = x.dim() - 2
    strides = _ints(a.get("strides")) or [1] * nd
    dil = _ints(a.get("dilations")) or [1] * nd
    pads = _ints(a.get("pads")) or [0] * (2 * nd)
    out_pad = _ints(a.get("output_padding")) or [0] * nd
    group = int(a.get("group", 1))
    if a.get("auto_pad", "NOTSET") not in ("NOTSET", b"NOTSET"):
        raise InvalidAttribute("ConvTranspose: auto_pad other than NOTSET is not supported")
    if pads[:nd] != pads[nd:]:
        raise InvalidAttribute("ConvTranspose: asymmetric pads are not supported")
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}.get(nd)
    if fn is None:
        raise InvalidGraph(f"ConvTranspose over {nd} spatial dimensions")
    want = _ints(a.get("output_shape"))
    if want:
        # output_shape overrides output_padding: out = stride (in - 1) + output_padding + dilation (k - 1) + 1 - 2 pad
        if len(want) != nd:
            raise InvalidAttribute(f"ConvTranspose: output_shape has {len(want)} entries for {nd} spatial dimensions")
        out_pad = []
        for d in range(nd):
            base = strides[d] * (x.shape[2 + d] - 1) + dil[d] * (w.shape[2 + d] - 1) + 1 - 2 * pads[d]
            extra = want[d] - base
            if extra < 0 or extra >= max(strides[d], dil[d]):
                raise InvalidAttribute(f"ConvTranspose: output_shape {want} is not reachable with pads {pads} "
                                       f"(dimension {d} would need output_padding {extra})")
            out_pad.append(extra)
    return [fn(x, w, b, stride=strides, padding=pads[:nd], output_padding=out_pad, groups=group, dilation=dil)]


@op("DepthToSpace", 1)
def _depth_to_space(i, a, c):
    x, bs = i[0], int(a["blocksize"])
    n, ch, h, w = x.shape
    mode = a.get("mode", "DCR")
    mode = mode.decode() if isinstance(mode, bytes) else mode
    if mode == "DCR":
        y = x.reshape(n, bs, bs, ch // (bs * bs), h, w).permute(0, 3, 4, 1, 5, 2)
    else:
        y = x.reshape(n, ch // (bs * bs), bs, bs, h, w).permute(0, 1, 4, 2, 5, 3)
    return [y.reshape(n, ch // (bs * bs), h * bs, w * bs)]


@op("SpaceToDepth", 1)
def _space_to_depth(i, a, c):
    x, bs = i[0], int(a["blocksize"])
    n, ch, h, w = x.shape
    y = x.reshape(n, ch, h // bs, bs, w // bs, bs).permute(0, 3, 5, 1, 2, 4)
    return [y.reshape(n, ch * bs * bs, h // bs, w // bs)]


@op("Resize", 1, 4)
def _resize(i, a, c):
    x = i[0]
    scales = i[2] if len(i) > 2 and i[2] is not None and i[2].numel() else None
    sizes = i[3] if len(i) > 3 and i[3] is not None and i[3].numel() else None
    mode = a.get("mode", "nearest")
    mode = mode.decode() if isinstance(mode, bytes) else mode
    ctm = a.get("coordinate_transformation_mode", "half_pixel")
    ctm = ctm.decode() if isinstance(ctm, bytes) else ctm
    nd = x.dim() - 2
    if sizes is not None:
        size = _ints(sizes)[-nd:]
    elif scales is not None:
        size = [int(math.floor(d * float(s))) for d, s in zip(x.shape[-nd:], scales.reshape(-1).tolist()[-nd:])]
    else:
        raise InvalidGraph("Resize needs scales or sizes")
    if mode == "nearest":
        # ONNX default rounding (round_prefer_floor on half_pixel / asymmetric) differs from torch's floor only on exact
        # halves; integer scale factors, the common case, agree
        return [F.interpolate(x, size=size, mode="nearest" if ctm == "asymmetric" else "nearest-exact")]
    tmode = {1: "linear", 2: "bilinear", 3: "trilinear"}[nd] if mode == "linear" else "bicubic"
    if ctm not in ("half_pixel", "pytorch_half_pixel", "align_corners"):
        raise InvalidAttribute(f"Resize: coordinate_transformation_mode {ctm} is not supported for {mode}")
    return [F.interpolate(x, size=size, mode=tmode, align_corners=(ctm == "align_corners"))]


# ------------------------------------------------------------------------------ indexing
@op("GatherElements", 2)
def _gather_elements(i, a, c):
    x, idx = i
    axis = int(a.get("axis", 0))
    idx = idx.to(torch.int64)
    idx = torch.where(idx < 0, idx + x.shape[axis], idx)
    return [torch.gather(x, axis, idx)]


@op("ScatterElements", 3)
def _scatter_elements(i, a, c):
    x, idx, upd = i
    axis = int(a.get("axis", 0))
    red = a.get("reduction", "none")
    red = red.decode() if isinstance(red, bytes) else red
    idx = idx.to(torch.int64)
    idx = torch.where(idx < 0, idx + x.shape[axis], idx)
    if red == "none":
        return [x.scatter(axis, idx, upd)]
    tred = {"add": "sum", "mul": "prod", "max": "amax", "min": "amin"}.get(red)
    if tred is None:
        raise InvalidAttribute(f"ScatterElements: reduction {red}")
    return [x.scatter_reduce(axis, idx, upd, tred, include_self=True)]


@op("GatherND", 2)
def _gather_nd(i, a, c):
    x, idx = i[0], i[1].to(torch.int64)
    if int(a.get("batch_dims", 0)):
        raise InvalidAttribute("GatherND: batch_dims > 0 is not supported")
    k = idx.shape[-1]
    idx = torch.where(idx < 0, idx + torch.tensor(x.shape[:k], device=idx.device), idx)
    return [x[tuple(idx[..., j] for j in range(k))]]


@op("ScatterND", 3)
def _scatter_nd(i, a, c):
    x, idx, upd = i[0].clone(), i[1].to(torch.int64), i[2]
    k = idx.shape[-1]
    red = a.get("reduction", "none")
    red = red.decode() if isinstance(red, bytes) else red
    key = tuple(idx[..., j] for j in range(k))
    if red == "none":
        x[key] = upd
    elif red == "add":
        x.index_put_(key, upd, accumulate=True)
    else:
        raise InvalidAttribute(f"ScatterND: reduction {red}")
    return [x]


@op("OneHot", 3)
def _one_hot(i, a, c):
    idx, depth, values = i[0].to(torch.int64), int(_ints(i[1])[0]), i[2]
    axis = int(a.get("axis", -1))
    idx = torch.where(idx < 0, idx + depth, idx)
    valid = (idx >= 0) & (idx < depth)
    hot = F.one_hot(idx.clamp(0, depth - 1), depth).to(torch.bool) & valid.unsqueeze(-1)
    out = torch.where(hot, values[1], values[0])
    if axis != -1 and axis != out.dim() - 1:
        out = out.movedim(-1, axis if axis >= 0 else axis + out.dim())
    return [out]


@op("NonZero", 1)
def _nonzero(i, a, c):
    return [torch.nonzero(i[0]).t().contiguous().to(torch.int64)]


@op("Trilu", 1, 2)
def _trilu(i, a, c):
    k = int(_ints(i[1])[0]) if len(i) > 1 and i[1] is not None else 0
    return [torch.triu(i[0], k) if int(a.get("upper", 1)) else torch.tril(i[0], k)]


@op("Size", 1)
def _size(i, a, c):
    return [torch.tensor(i[0].numel(), dtype=torch.int64, device=i[0].device)]


@op("EyeLike", 1)
def _eye_like(i, a, c):
    x = i[0]
    from .dtypes import DataTypeMapper
    dt = DataTypeMapper.from_onnx(int(a["dtype"])).torch if "dtype" in a else x.dtype
    k = int(a.get("k", 0))
    return [torch.ones(x.shape[0], x.shape[1], dtype=dt, device=x.device).triu(k).tril(k)]


@op("Einsum", 1, None)
def _einsum(i, a, c):
    eq = a["equation"]
    return [torch.einsum(eq.decode() if isinstance(eq, bytes) else eq, *i)]


# ------------------------------------------------------------------------------ quantisation
def _qparams(x, scale, zp, axis):
    if scale.dim() == 0 or scale.numel() == 1:
        return scale.reshape(()), (zp.reshape(()) if zp is not None else None)
    shape = [1] * x.dim()
    shape[axis] = -1
    return scale.reshape(shape), (zp.reshape(shape) if zp is not None else None)


@op("QuantizeLinear", 2, 3)
def _quantize_linear(i, a, c):
    x, scale = i[0], i[1]
    zp = i[2] if len(i) > 2 else None
    scale_b, zp_b = _qparams(x, scale, zp, int(a.get("axis", 1)))
    dt = zp.dtype if zp is not None else torch.uint8
    lo, hi = (0, 255) if dt == torch.uint8 else (-128, 127)
    q = torch.round(x / scale_b)
    if zp_b is not None:
        q = q + zp_b.to(q.dtype)
    return [q.clamp(lo, hi).to(dt)]


@op("DequantizeLinear", 2, 3)
def _dequantize_linear(i, a, c):
    x, scale = i[0], i[1]
    zp = i[2] if len(i) > 2 else None
    scale_b, zp_b = _qparams(x, scale, zp, int(a.get("axis", 1)))
    v = x.to(torch.float32)
    if zp_b is not None:
        v = v - zp_b.to(torch.float32)
    return [(v * scale_b).to(scale.dtype)]


# ------------------------------------------------------------------------------ recurrent layers
# X [seq, batch, input] (layout 0) or [batch, seq, input] (layout 1); W [dirs, G*hidden, input]; R [dirs, G*hidden, hidden];
# B [dirs, 2*G*hidden] (input bias then recurrent bias); default activations only; no peepholes, no clipping.
def _str_attr(a, key, default):
    v = a.get(key, default)
    return v.decode() if isinstance(v, bytes) else v


def _recurrent(kind: str, gates: int):
    def run(i, a, c):
        x, w, r = i[0], i[1], i[2]
        b = i[3] if len(i) > 3 else None
        seq_lens = i[4] if len(i) > 4 else None
        h0 = i[5] if len(i) > 5 else None
        c0 = i[6] if kind == "LSTM" and len(i) > 6 else None
        if kind == "LSTM" and len(i) > 7 and i[7] is not None:
            raise InvalidAttribute("LSTM: peephole weights are not supported")
        if seq_lens is not None:
            raise InvalidAttribute(f"{kind}: sequence_lens is not supported (pad-free batches only)")
        if a.get("activations") and kind != "RNN":
            raise InvalidAttribute(f"{kind}: only the default activations are supported")
        if a.get("clip") is not None:
            raise InvalidAttribute(f"{kind}: clip is not supported")
        hidden = int(a["hidden_size"])
        direction = _str_attr(a, "direction", "forward")
        layout = int(a.get("layout", 0))
        if layout == 1:
            x = x.transpose(0, 1)
            h0 = h0.transpose(0, 1) if h0 is not None else None
            c0 = c0.transpose(0, 1) if c0 is not None else None
        seq, batch = x.shape[0], x.shape[1]
        dirs = 2 if direction == "bidirectional" else 1
        if w.shape[0] != dirs:
            raise InvalidGraph(f"{kind}: W has {w.shape[0]} directions, attribute direction={direction}")
        act = torch.tanh
        if kind == "RNN" and a.get("activations"):
            names = [n.decode() if isinstance(n, bytes) else n for n in a["activations"]]
            if any(n not in ("Tanh", "Relu") for n in names):
                raise InvalidAttribute("RNN: activations other than Tanh / Relu are not supported")
            act = torch.relu if names[0] == "Relu" else torch.tanh
        lbr = int(a.get("linear_before_reset", 0))
        ys, hs, cs = [], [], []
        for d in range(dirs):
            wd, rd = w[d], r[d]
            wb = b[d, :gates * hidden] if b is not None else None
            rb = b[d, gates * hidden:] if b is not None else None
            h = h0[d] if h0 is not None else x.new_zeros(batch, hidden)
            cell = c0[d] if c0 is not None else x.new_zeros(batch, hidden)
            reverse = direction == "reverse" or d == 1
            steps = range(seq - 1, -1, -1) if reverse else range(seq)
            out = [None] * seq
            xw = F.linear(x, wd, wb)                              # every time step's input projection at once
            for t_ in steps:
                if kind == "LSTM":                                # gate order i, o, f, c
                    g = xw[t_] + F.linear(h, rd, rb)
                    gi, go, gf, gc = g.chunk(4, -1)
                    cell = torch.sigmoid(gf) * cell + torch.sigmoid(gi) * torch.tanh(gc)
                    h = torch.sigmoid(go) * torch.tanh(cell)
                elif kind == "GRU":                               # gate order z, r, h
                    xz, xr, xh = xw[t_].chunk(3, -1)
                    rz, rr, rh = rd.chunk(3, 0)
                    bz, br, bh = rb.chunk(3, -1) if rb is not None else (None, None, None)
                    z = torch.sigmoid(xz + F.linear(h, rz, bz))
                    rg = torch.sigmoid(xr + F.linear(h, rr, br))
                    if lbr:
                        cand = torch.tanh(xh + rg * F.linear(h, rh, bh))
                    else:
                        cand = torch.tanh(xh + F.linear(rg * h, rh, bh))
                    h = (1 - z) * cand + z * h
                else:
                    h = act(xw[t_] + F.linear(h, rd, rb))
                out[t_] = h
            ys.append(torch.stack(out, 0))
            hs.append(h)
            cs.append(cell)
        y = torch.stack(ys, 1)                                    # [seq, dirs, batch, hidden]
        yh = torch.stack(hs, 0)
        if layout == 1:
            y, yh = y.permute(2, 0, 1, 3), yh.transpose(0, 1)
        outs = [y, yh]
        if kind == "LSTM":
            yc = torch.stack(cs, 0)
            outs.append(yc.transpose(0, 1) if layout == 1 else yc)
        return outs
    return run


op("LSTM", 3, 8)(_recurrent("LSTM", 4))
op("GRU", 3, 6)(_recurrent("GRU", 3))
op("RNN", 3, 6)(_recurrent("RNN", 1))


# ------------------------------------------------------------------------------ integer matmul (QOperator format)
def _zp(t, like_rows: bool):
    """Zero point as an int32 tensor broadcastable against a [.., M, K] (rows) or [.., K, N] (columns) operand."""
    if t is None:
        return 0
    z = t.to(torch.int32)
    if z.dim() == 0 or z.numel() == 1:
        return z.reshape(())
    return z.reshape(-1, 1) if like_rows else z.reshape(1, -1)


@op("MatMulInteger", 2, 4)
def _matmul_integer(i, a, c):
    x, w = i[0].to(torch.int32), i[1].to(torch.int32)
    xz = _zp(i[2] if len(i) > 2 else None, True)
    wz = _zp(i[3] if len(i) > 3 else None, False)
    # int32 matmul is not available on every device: accumulate in float64, exact up to 2^53
    return [((x - xz).to(torch.float64) @ (w - wz).to(torch.float64)).to(torch.int32)]


@op("DynamicQuantizeLinear", 1)
def _dynamic_quantize_linear(i, a, c):
    x = i[0].to(torch.float32)
    lo, hi = torch.clamp(x.min(), max=0.0), torch.clamp(x.max(), min=0.0)
    scale = (hi - lo) / 255.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    zp = torch.clamp(torch.round(-lo / scale), 0, 255)
    y = torch.clamp(torch.round(x / scale) + zp, 0, 255).to(torch.uint8)
    return [y, scale.reshape(()), zp.to(torch.uint8).reshape(())]


@op("QLinearMatMul", 8)
def _qlinear_matmul(i, a, c):
    xa, sa, za, xb, sb, zb, sy, zy = i
    acc = (xa.to(torch.int32) - _zp(za, True)).to(torch.float64) @ (xb.to(torch.int32) - _zp(zb, False)).to(torch.float64)
    sa_, sb_ = sa.to(torch.float64), sb.to(torch.float64)
    if sa_.numel() > 1:
        sa_ = sa_.reshape(-1, 1)
    if sb_.numel() > 1:
        sb_ = sb_.reshape(1, -1)
    y = torch.round(acc * sa_ * sb_ / sy.to(torch.float64)) + zy.to(torch.float64)
    lo, hi = (0, 255) if zy.dtype == torch.uint8 else (-128, 127)
    return [y.clamp(lo, hi).to(zy.dtype)]


def _conv_args(a, nd):
    pads = _ints(a.get("pads")) or [0] * (2 * nd)
    if pads[:nd] != pads[nd:]:
        raise InvalidAttribute("integer convolution: asymmetric pads are not supported")
    if a.get("auto_pad", "NOTSET") not in ("NOTSET", b"NOTSET"):
        raise InvalidAttribute("integer convolution: auto_pad other than NOTSET is not supported")
    return dict(stride=_ints(a.get("strides")) or [1] * nd, padding=pads[:nd],
                dilation=_ints(a.get("dilations")) or [1] * nd, groups=int(a.get("group", 1)))


def _int_conv(x, w, xz, wz, a):
    """Exact integer convolution of (x - xz) with (w - wz[per output channel]) computed in float64."""
    nd = x.dim() - 2
    xs = x.to(torch.float64) - (float(xz.reshape(-1)[0]) if xz is not None else 0.0)
    ws = w.to(torch.float64)
    if wz is not None:
        ws = ws - wz.to(torch.float64).reshape(-1, *([1] * (w.dim() - 1)))
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
    # zero padding must add (x - xz) = 0, i.e. pad the shifted tensor, which conv's own padding does
    return fn(xs, ws, None, **_conv_args(a, nd))


@op("ConvInteger", 2, 4)
def _conv_integer(i, a, c):
    y = _int_conv(i[0], i[1], i[2] if len(i) > 2 else None, i[3] if len(i) > 3 else None, a)
    return [y.to(torch.int32)]


@op("QLinearConv", 8, 9)
def _qlinear_conv(i, a, c):
    x, xs, xz, w, ws, wz, ys, yz = i[:8]
    bias = i[8] if len(i) > 8 else None
    acc = _int_conv(x, w, xz, wz, a)
    if bias is not None:                                         # int32, in units of x_scale * w_scale
        acc = acc + bias.to(torch.float64).reshape(1, -1, *([1] * (acc.dim() - 2)))
    wsc = ws.to(torch.float64)
    wsc = wsc.reshape(1, -1, *([1] * (acc.dim() - 2))) if wsc.numel() > 1 else wsc
    y = torch.round(acc * xs.to(torch.float64) * wsc / ys.to(torch.float64)) + yz.to(torch.float64)
    lo, hi = (0, 255) if yz.dtype == torch.uint8 else (-128, 127)
    return [y.clamp(lo, hi).to(yz.dtype)]
